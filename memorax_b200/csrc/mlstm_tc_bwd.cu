// Backward of the chunked tensor-core mLSTM (mlstm_tc.cu) on the sm_100a tensor cores.
//
// One CTA (256 threads, two warpgroups) owns one (batch, head) sequence and walks its 64-token chunks right to
// left, carrying G^T = (dL/d[C | n])^T in tensor memory (fp32); the state entering each chunk and the stabiliser
// of every step come from the forward call's residuals.  The stabiliser m is a gauge: every decay factor below
// contains it, but the read-out depends on it only through eps exp(m_t) in the denominator, so the factors are
// differentiated with m held fixed and that one explicit dependence is added separately.  Per chunk, with the
// forward kernel's D, w, kappa, delta,  den_t = max(|qn_t|, exp(-m_t)) + eps:
//   phase 1 (independent MMAs):  P = Q K^T,  dA = dH V^T,  R = dH S_in,  Y = K [G | gn]
//   epilogue 1 (four threads per query row, 16 keys each):
//     P~_tj = D_tj P_tj        qn_t = sum_j P~_tj + w_t q_t.n_in        don_t = sum_j P~_tj dA_tj + w_t q_t.R_t
//     dden_t = -don_t / den_t^2     dqn_t = [|qn_t| >= exp(-m_t)] sign(qn_t) dden_t
//     Pn_tj = P~_tj / den_t         dP~_tj = dA_tj / den_t + dqn_t        dA'_tj = D_tj dP~_tj
//     dOs_t = w_t [dh_t / den_t | dqn_t]
//     gate terms:  E_tj = dP~_tj P~_tj,  Ew_t = w_t (q_t.R_t / den_t + dqn_t q_t.n_in),
//                  Ek_j = kappa_j [v_j | 1] . Y_j,  Ed = delta <G, S_in>,  dm_t = eps dden_t
//   phase 2:  dQ = dA' K + dOs [S_in | n_in]
//             dK = dA'^T Q + (kappa o [V | 1]) [G | gn]^T
//             dV = Pn^T dH + (kappa o K) G^T
//             [G | gn]^T = delta [G | gn]^T + Q^T dOs
//   gate gradients of the chunk (warp 1):
//     dcumf_t = sum_j E_tj - sum_i E_it + Ew_t - Ek_t,   dcumf_last += sum_j Ek_j + Ed
//     dli_j = sum_t E_tj + Ek_j,   dlf_s = sum_{t >= s} dcumf_t
//     and the explicit path: g_t = dm_t + [step t+1 took the forget branch] g_{t+1}, carried chunk to chunk;
//     a step that took the input branch (or a reset) sends g_t to dli_t, the others to dlf_t.
#include <cuda_bf16.h>

#include "linattn_common.cuh"
#include "mlstm_tc_common.cuh"
#include "mxk_common.cuh"
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace linattn;
using namespace mlstm_tc;

constexpr int kPanelsK = kPanels + 2;  // 80 columns: a K = 80 contraction needs whole K=16 steps
// 256 threads: two warpgroups that see the same TMEM lanes (warp w and warp w + 4 share a
// lane quarter) and split the columns of every row between them.
constexpr int kBwdThreads = 256;

struct BwdParams {
  const float* log_i; const float* log_f;     // (B,T,H)
  const float* m_steps;                       // (B,T,H) residual: the stabiliser after every step
  const float* m0;                            // (B,H) carried stabiliser, NULL = -1e9
  const float* c0; const float* n0;           // carried state (for dm0), NULL = zeros
  const float* c_last; const float* n_last;   // the forward call's next carry (for the gauge term of its cotangents)
  const uint4* chunk_states;
  const uint8_t* done;
  const float* dc_last; const float* dn_last; const float* dm_last;
  float* dlog_i; float* dlog_f;               // (B,T,H) out
  float* dc0; float* dn0; float* dm0;         // optional
  int* status;
  int B, T, H;
  float eps;
  int d;   // head dimension: a multiple of 8, at most kD; the tiles are kD wide, the rest zero
  CUtensorMap map_q, map_k, map_v, map_do;   // 64-token tiles as SW tiles
  CUtensorMap map_dq, map_dk, map_dv;        // the same for the outputs
};

struct GateGrads {
  float colpart[4][kC];    // sum over the 16 rows of a lane quarter of E_tj, per key j
  float ew[kC];            // Ew_t
  float rowsum[kC];        // sum_j E_tj
  float ekpart[2][kC];     // per warpgroup: partial Ek_j
  float dmexp[kC];         // dm_t = eps dden_t (plus the next carry's gauge term at the last step)
  float edpart[8];         // per warp: partial <G, S_in>
  float gauge[8];          // per warp: partial <dC_last, C_T> + <dn_last, n_T>, later <dC_0, C_0> + <dn_0, n_0>
};

struct BwdSmem {
  // 128-byte-swizzled row-major tiles (umma.cuh "SW tiles"), 8 KB each, 1024-byte aligned
  uint4 q[kPanels * kC];      // Q
  uint4 k[kPanels * kC];      // K
  uint4 v[kPanels * kC];      // V
  uint4 d_o[kPanels * kC];    // dH
  uint4 kk[kPanels * kC];     // kappa o K
  uint4 vk[kPanels * kC];     // kappa o V
  // panel format
  uint4 vkx[2 * kC];          // columns 64..79 of kappa o [V | 1 | 0]
  uint4 dos[kPanelsK * kC];   // w o [dH / den | dqn] | 0
  uint4 s[kPanelsK * kD];     // [C_in | n_in]^T | 0    [v/8][k]
  uint4 g[kPanelsK * kD];     // [G | gn]^T | 0         [v/8][k]
  uint4 pn[kPanels * kC];     // P~ / den               [j/8][t]
  uint4 dp[kPanels * kC];     // dA' = D o dP~          [j/8][t]
  float xch[2][2][kC];        // per warpgroup: partial qn and don of every query row
  ChunkGates gates;
  GateGrads gg;
  uint64_t bar[2];
  uint64_t bar_load;
  uint32_t tmem;
};
static_assert(sizeof(BwdSmem) <= 113 * 1024, "two CTAs per SM");

// 256 TMEM columns per CTA (two CTAs per SM).  M = 64 accumulators use 16 of a warp's 32 TMEM lanes, so lanes
// 0..15 ("lower" threads) and 16..31 ("upper" threads) hold different matrices in the same columns:
//   columns   0.. 63   first P (0..31) and dA (32..63), each issued as two N = 32 halves: keys 0..31 in the lower
//                      lanes, keys 32..63 in the upper lanes, so that both half-warps own 32 keys of the same query
//                      row; later dQ (lower) and dK (upper)
//   columns  64..135   lower: dV                  upper: [G | gn]^T (persistent)
//   columns 136..167   R, state features 0..31 in the lower lanes, 32..63 in the upper lanes
//   columns 168..239   lower: Y = K [G | gn]
// Within a half-warp's 32 columns, warpgroup 0 takes the first 16 and warpgroup 1 the rest.
#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_mtcb_phase_cycles[16];
namespace {
#define MXK_TMB(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_mtcb_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_TMB(i) do {} while (0)
#endif
constexpr uint32_t kBwdTmemCols = 256;
constexpr uint32_t kUpper = 16u << 16;
constexpr uint32_t kColLo = 0, kColHi = 64, kColP = 0, kColA = 32, kColR = 136, kColY = 168;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }

// Sum of x over the 16 lanes of a half-warp, for 16 values at once: after four exchange steps lane i of the
// half holds the total of value i (15 shuffles instead of 64).
__device__ __forceinline__ float half_warp_reduce_scatter(float* a, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float send = (lane & 8) ? a[i] : a[i + 8], keep = (lane & 8) ? a[i + 8] : a[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = (lane & 4) ? a[i] : a[i + 4], keep = (lane & 4) ? a[i + 4] : a[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = (lane & 2) ? a[i] : a[i + 2], keep = (lane & 2) ? a[i + 2] : a[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const float send = (lane & 1) ? a[0] : a[1], keep = (lane & 1) ? a[1] : a[0];
  return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

// Gate gradients of one chunk, by one warp (lane l owns tokens 2l, 2l + 1); `carry` is the explicit-path cotangent
// flowing in from the chunk to the right (already multiplied by that chunk's first forget flag) and is replaced by
// the one flowing out to the left.
__device__ __forceinline__ void chunk_gate_grads(const ChunkGates& g, const GateGrads& gg, uint64_t dm, float m_in, float ed,
                                                 float& carry, float* dli_out, float* dlf_out, int t0, int T, int H, int lane) {
  const int a = 2 * lane, b = a + 1;
  float ek_a = gg.ekpart[0][a] + gg.ekpart[1][a], ek_b = gg.ekpart[0][b] + gg.ekpart[1][b];
  float col_a = (gg.colpart[0][a] + gg.colpart[1][a]) + (gg.colpart[2][a] + gg.colpart[3][a]);
  float col_b = (gg.colpart[0][b] + gg.colpart[1][b]) + (gg.colpart[2][b] + gg.colpart[3][b]);
  float dc_a = gg.rowsum[a] - col_a + gg.ew[a] - ek_a, dc_b = gg.rowsum[b] - col_b + gg.ew[b] - ek_b;
  float ek_sum = ek_a + ek_b;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) ek_sum += __shfl_xor_sync(0xffffffffu, ek_sum, off);
  if (lane == 31) dc_b += ek_sum + ed;      // cumf_T = cumf of the chunk's last slot
  // dlf_s = sum_{t >= s} dcumf_t: inclusive suffix sum
  float suf = dc_a + dc_b;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float o = __shfl_down_sync(0xffffffffu, suf, off);
    if (lane + off < 32) suf += o;
  }
  float dlf_a = suf, dlf_b = suf - dc_a;
  float dli_a = col_a + ek_a, dli_b = col_b + ek_b;
  // explicit path: G_t = dm_t + fg_{t+1} G_{t+1} with fg_t = [step t took the forget branch] and the carry (already
  // multiplied by the flag of the first step to the right) entering after the last token.  What a lane hands to
  // its left neighbour, Z_l = fg_a G_a, is affine in what it receives: Z_l = X_l + A_l Z_{l+1}; suffix scan of the maps.
  const float m_pa = lane > 0 ? g.m[a - 1] : m_in;   // stabiliser before token a
  const float fg_a = (!((dm >> a) & 1ull) && m_pa + g.lf[a] >= g.li[a]) ? 1.f : 0.f;
  const float fg_b = (!((dm >> b) & 1ull) && g.m[a] + g.lf[b] >= g.li[b]) ? 1.f : 0.f;
  const float xa = gg.dmexp[a], xb = gg.dmexp[b];
  float A = fg_a * fg_b, X = fg_a * fmaf(fg_b, xb, xa);
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float Ao = __shfl_down_sync(0xffffffffu, A, off), Xo = __shfl_down_sync(0xffffffffu, X, off);
    if (lane + off < 32) { X = fmaf(A, Xo, X); A *= Ao; }
  }
  const float Xn = __shfl_down_sync(0xffffffffu, X, 1), An = __shfl_down_sync(0xffffffffu, A, 1);
  const float R = lane < 31 ? fmaf(An, carry, Xn) : carry;
  const float Gb = xb + R, Ga = fmaf(fg_b, Gb, xa);
  const float carry_out = __shfl_sync(0xffffffffu, fmaf(A, carry, X), 0);
  dli_a += (1.f - fg_a) * Ga; dlf_a += fg_a * Ga;
  dli_b += (1.f - fg_b) * Gb; dlf_b += fg_b * Gb;
  carry = carry_out;
  const int ta = t0 + a;
  if (ta < T) { dli_out[static_cast<size_t>(ta) * H] = dli_a; dlf_out[static_cast<size_t>(ta) * H] = dlf_a; }
  if (ta + 1 < T) { dli_out[static_cast<size_t>(ta + 1) * H] = dli_b; dlf_out[static_cast<size_t>(ta + 1) * H] = dlf_b; }
}

__global__ void __launch_bounds__(kBwdThreads, 2) mlstm_tc_bwd_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;   // warpgroup
  const int qw = warp & 3;    // TMEM lane quarter of this warp
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const bool upper = lane >= 16;
  const int row = qw * 16 + (lane & 15);
  const int nchunks = (p.T + kC - 1) / kC;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  const int hd = p.d;

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init(&sm.bar_load, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kBwdTmemCols);
  // zero padding panels that never change (columns 72..79 of the 80-wide operands)
  if (tid < kC) {
    sm.vkx[kC + tid] = zero4;
    sm.dos[(kPanelsK - 1) * kC + tid] = zero4;
    sm.s[(kPanelsK - 1) * kD + tid] = zero4;
    sm.g[(kPanelsK - 1) * kD + tid] = zero4;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(qw * 32) << 16);

  auto issue_chunk_loads = [&](int cc) {
    fence_smem_to_async();   // earlier generic-proxy accesses to the buffers come first
    tma::expect_bytes(&sm.bar_load, (4 * kPanels * kC + kPanelsX * kD) * 16);
    tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.v, &p.map_v, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.d_o, &p.map_do, &sm.bar_load, cc * kC, h, b);
    tma::load_bulk(sm.s, p.chunk_states + (static_cast<size_t>(bh) * nchunks + cc) * (kPanelsX * kD),
                   kPanelsX * kD * 16, &sm.bar_load);
    if (cc > 0) {   // the chunk after it (walking right to left): into L2 now, so that its loads hit there
      tma::prefetch_plain_tile(&p.map_q, (cc - 1) * kC, h, b);
      tma::prefetch_plain_tile(&p.map_k, (cc - 1) * kC, h, b);
      tma::prefetch_plain_tile(&p.map_v, (cc - 1) * kC, h, b);
      tma::prefetch_plain_tile(&p.map_do, (cc - 1) * kC, h, b);
      tma::prefetch_bulk(p.chunk_states + (static_cast<size_t>(bh) * nchunks + cc - 1) * (kPanelsX * kD), kPanelsX * kD * 16);
    }
  };
  if (tid == 0) issue_chunk_loads(nchunks - 1);

  // Cotangent of the next carry -> TMEM (upper lanes) and its bf16 operand copy (upper thread `row` owns
  // G^T[row][.] = dC[row][.], gn_row; warpgroup 0 takes value columns 0..31, warpgroup 1 columns 32..63 and gn),
  // and the gauge term <dC_last, C_T> + <dn_last, n_T> of the explicit path.
  const int gp0 = wg ? 4 : 0, gpn = wg ? 5 : 4;   // this warpgroup's panels of the 72-column accumulator
  {
    const bool mine = upper && row < hd;
    const float* gs = (p.dc_last && mine) ? p.dc_last + (static_cast<size_t>(bh) * hd + row) * hd : nullptr;
    const float* cs = (p.c_last && mine) ? p.c_last + (static_cast<size_t>(bh) * hd + row) * hd : nullptr;
    float vals[40];   // all loads first: the TMEM stores below are compiler memory barriers
    float gauge = 0.f;
#pragma unroll
    for (int i = 0; i < 40; ++i) {
      const int vcol = gp0 * 8 + i;
      float x = 0.f;
      if (mine && i < gpn * 8) {
        if (vcol < kD) {
          x = (gs && vcol < hd) ? gs[vcol] : 0.f;
          if (cs && vcol < hd) gauge = fmaf(x, cs[vcol], gauge);
        } else if (vcol == kD) {
          x = p.dn_last ? p.dn_last[static_cast<size_t>(bh) * hd + row] : 0.f;
          if (p.n_last) gauge = fmaf(x, p.n_last[static_cast<size_t>(bh) * hd + row], gauge);
        }
      }
      vals[i] = x;
    }
#pragma unroll
    for (int pn = 0; pn < 5; ++pn) {
      if (pn < gpn) {
        tmem_st8(lane_base + kColHi + (gp0 + pn) * 8, vals + pn * 8);
        if (upper) sm.g[(gp0 + pn) * kD + row] = pack8_bf16(vals + pn * 8);
      }
    }
    tmem_st_wait();
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) gauge += __shfl_xor_sync(0xffffffffu, gauge, off);
    if (lane == 0) sm.gg.gauge[warp] = gauge;
  }

  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint32_t id_kk = idesc_bf16(kC, kC, false, false);   // A, B contract over columns
  const uint32_t id_km = idesc_bf16(kC, kC, false, true);    // B contracts over rows
  const uint32_t id_mm = idesc_bf16(kC, kC, true, true);
  const uint32_t id_g = idesc_bf16(kD, kDX, true, true);
  const uint32_t id_y = idesc_bf16(kC, kDX, false, true);
  bool timed_out = false;
  DoneFlags done_flags = load_done_flags(drow, (nchunks - 1) * kC, p.T, lane);
  LaneGates lane_gates = load_lane_gates(p.log_i, p.log_f, b, h, (nchunks - 1) * kC, p.T, p.H, lane);   // used by warp 1
  auto load_m_in = [&](int cc) -> float {   // the stabiliser entering chunk cc
    if (cc <= 0) return p.m0 ? p.m0[bh] : -1e9f;
    return __ldg(p.m_steps + (static_cast<size_t>(b) * p.T + cc * kC - 1) * p.H + h);
  };
  float m_in_next = load_m_in(nchunks - 1);
  float carry = 0.f;   // explicit-path cotangent entering from the right (meaningful in warp 1)
  // Warp 1 computes a chunk's gate factors one chunk ahead: for the last chunk here, afterwards (behind that chunk's
  // gate gradients) while the second MMA group of the chunk to the right runs.
  if (warp == 1) {
    chunk_gate_scan(sm.gates, lane_gates, done_mask_from_flags(done_flags), m_in_next, 0.f, lane, (nchunks - 1) & 1);
    lane_gates = load_lane_gates(p.log_i, p.log_f, b, h, (nchunks - 2) * kC, p.T, p.H, lane);
  }
  float* dli_out = p.dlog_i + static_cast<size_t>(b) * p.T * p.H + h;
  float* dlf_out = p.dlog_f + static_cast<size_t>(b) * p.T * p.H + h;

#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif
  for (int it = 0; it < nchunks; ++it) {
    MXK_TMB(0);
    const int c = nchunks - 1 - it;
    const int t0 = c * kC;
    const int valid = min(kC, p.T - t0);
    const uint64_t dm = done_mask_from_flags(done_flags);
    done_flags = load_done_flags(drow, t0 - kC, p.T, lane);   // the next (earlier) chunk's flags
    const bool has_reset = dm != 0ull;
    const float m_in = m_in_next;
    m_in_next = load_m_in(c - 1);
    mbar_wait_flag(&sm.bar_load, it & 1, timed_out);
    MXK_TMB(1);
    if (tid == 0) tma::wait_group_read<0>();   // the previous chunk's output tiles have left their staging buffers
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    MXK_TMB(2);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand aq = sw_operand(smem_u32(sm.q), false), bk = sw_operand(smem_u32(sm.k), false);
      const Operand ado = sw_operand(smem_u32(sm.d_o), false), bv = sw_operand(smem_u32(sm.v), false);
      const Operand bs{smem_u32(sm.s), kD, false};
      const uint32_t id_half = idesc_bf16(kC, 32, false, false);
      // rows 32..63 of an SW tile start 32 lines further on
      const Operand bk_hi = sw_operand(smem_u32(sm.k) + 32 * 128, false), bv_hi = sw_operand(smem_u32(sm.v) + 32 * 128, false);
      const Operand bs_hi{smem_u32(sm.s) + 32 * 16, kD, false};
      gemm<kD / 16>(tmem + kColP, aq, bk, id_half, false, leader);                 // P,  keys 0..31
      gemm<kD / 16>(tmem + kUpper + kColP, aq, bk_hi, id_half, false, leader);     // P,  keys 32..63
      gemm<kD / 16>(tmem + kColA, ado, bv, id_half, false, leader);                // dA, keys 0..31
      gemm<kD / 16>(tmem + kUpper + kColA, ado, bv_hi, id_half, false, leader);    // dA, keys 32..63
      gemm<kD / 16>(tmem + kColR, ado, bs, id_half, false, leader);                // R,  features 0..31
      gemm<kD / 16>(tmem + kUpper + kColR, ado, bs_hi, id_half, false, leader);    // R,  features 32..63
      gemm<kD / 16>(tmem + kColY, sw_operand(smem_u32(sm.k), false), Operand{smem_u32(sm.g), kD, true}, id_y, false, leader);   // Y = K [G | gn]
      if (leader) commit(&sm.bar[0]);
    }
    const float delta = sm.gates.delta;
    // ---- while the first MMA group runs: what depends only on the tiles, the gates and the G of the previous
    //      chunk (none of it on this group's products, none of it in the columns the group writes) ----
    {
      // kappa-scaled copies of K and V (SW tiles: physical vector index serves, row = vid >> 3) and of the "1" column
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int vid = r * kBwdThreads + tid;
        const float kap = sm.gates.kappa[vid >> 3];
        float f[8];
        unpack8_bf16(sm.k[vid], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= kap;
        sm.kk[vid] = pack8_bf16(f);
        unpack8_bf16(sm.v[vid], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= kap;
        sm.vk[vid] = pack8_bf16(f);
      }
      if (tid < kC) sm.vkx[tid] = make_uint4(pack_bf16(tid < valid ? sm.gates.kappa[tid] : 0.f, 0.f), 0, 0, 0);
      // G <- delta G in tensor memory (upper lanes; the lower lanes of the warp-wide store rewrite a dead dV), and
      // Ed = delta <G, S_in> before that
      {
        float acc[40];
        if (wg == 0) tmem_ld_row<32>(lane_base + kColHi, acc);
        else tmem_ld_row<40>(lane_base + kColHi + 32, acc);
        float ed = 0.f;
        if (upper) {
#pragma unroll
          for (int pn = 0; pn < 5; ++pn) {
            if (pn < gpn) {
              float f[8];
              unpack8_bf16(sm.s[(gp0 + pn) * kD + row], f);
#pragma unroll
              for (int e = 0; e < 8; ++e) ed = fmaf(acc[pn * 8 + e], f[e], ed);
            }
          }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ed += __shfl_xor_sync(0xffffffffu, ed, off);
        if (lane == 0) sm.gg.edpart[warp] = ed;
        if (!has_reset) {
#pragma unroll
          for (int i = 0; i < 40; ++i) acc[i] *= upper ? delta : 1.f;
#pragma unroll
          for (int pn = 0; pn < 5; ++pn)
            if (pn < gpn) tmem_st8(lane_base + kColHi + (gp0 + pn) * 8, acc + pn * 8);
          tmem_st_wait();
        }
      }
    }
    mbar_wait_flag(&sm.bar[0], it & 1, timed_out);
    fence_after_sync();
    MXK_TMB(3);

    // ---- epilogue 1: the four threads of a query row (two half-warps x two warpgroups) each cover 16 keys /
    //      state features; qn and don are completed through shared memory ----
    {
      const int lo = row_first_key(dm, row);
      const int j0 = (upper ? 32 : 0) + wg * 16;   // first key / feature of this thread
      const int p0 = j0 >> 3;                      // and its first panel
      const float w = sm.gates.w[row], rt = sm.gates.rowterm2[row];
      float s_dot = 0.f, z_dot = 0.f;
      {
        float rr[16];
        tmem_ld_row<16>(lane_base + kColR + wg * 16, rr);
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
          float fq[8];
          unpack8_bf16(sm.q[sw_idx(row, p0 + pp)], fq);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int kk = (p0 + pp) * 8 + e;
            s_dot = fmaf(fq[e], rr[pp * 8 + e], s_dot);
            z_dot = fmaf(fq[e], bf16_lo(sm.s[kPanels * kD + kk].x), z_dot);
          }
        }
      }
      float pv[16], av[16], dw[16];
      tmem_ld_row<16>(lane_base + kColP + wg * 16, pv);
      tmem_ld_row<16>(lane_base + kColA + wg * 16, av);
      float qn = w * z_dot, don = w * s_dot;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int j = j0 + e;
        const bool m = (j >= lo && j <= row);
        dw[e] = m ? ex2_fast(rt + sm.gates.lic2[j]) : 0.f;
        pv[e] *= dw[e];                     // P~
        av[e] = m ? av[e] : 0.f;
        qn += pv[e];
        don = fmaf(pv[e], av[e], don);
      }
      // the inter-chunk parts of qn and don, summed over the row's four threads (for Ew)
      float z_all = z_dot, s_all = s_dot;
      z_all += __shfl_xor_sync(0xffffffffu, z_all, 16);
      s_all += __shfl_xor_sync(0xffffffffu, s_all, 16);
      qn += __shfl_xor_sync(0xffffffffu, qn, 16);
      don += __shfl_xor_sync(0xffffffffu, don, 16);
      if (!upper) {
        sm.xch[wg][0][row] = qn;
        sm.xch[wg][1][row] = don;
        sm.gg.colpart[wg][row] = z_all;      // borrowed for the exchange of the inter parts (rewritten below)
        sm.gg.colpart[2 + wg][row] = s_all;
      }
      MXK_TMB(4);
      __syncthreads();
      MXK_TMB(5);
      qn += sm.xch[wg ^ 1][0][row];
      don += sm.xch[wg ^ 1][1][row];
      z_all += sm.gg.colpart[wg ^ 1][row];
      s_all += sm.gg.colpart[2 + (wg ^ 1)][row];
      const float em = sm.gates.em[c & 1][row];
      const float den = fmaxf(fabsf(qn), em) + p.eps;
      const float inv = 1.f / den;
      const float dden = -don * inv * inv;
      const float dqn = fabsf(qn) >= em ? (qn > 0.f ? dden : (qn < 0.f ? -dden : 0.f)) : 0.f;
      float ecol[16];
#pragma unroll
      for (int jq = 0; jq < 2; ++jq) {
        float a[8], d8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int x = jq * 8 + e;
          const float dpt = fmaf(av[x], inv, dqn);     // dP~ (masked through pv / dw below)
          a[e] = pv[x] * inv;
          d8[e] = dw[x] * dpt;
          ecol[x] = pv[x] * dpt;                       // E_tj = dP~ P~ (zero outside the mask: P~ is)
        }
        sm.pn[(p0 + jq) * kC + row] = pack8_bf16(a);
        sm.dp[(p0 + jq) * kC + row] = pack8_bf16(d8);
      }
      MXK_TMB(6);
      __syncthreads();   // every thread has read the borrowed colpart slots
      MXK_TMB(7);
      {
        const float tot = half_warp_reduce_scatter(ecol, lane);
        sm.gg.colpart[qw][j0 + (lane & 15)] = tot;
      }
      // scaled dH rows: two of the eight panels per thread, the extra column by one of the four
      const float sc = w * inv;
#pragma unroll
      for (int pp = 0; pp < 2; ++pp) {
        float f[8];
        unpack8_bf16(sm.d_o[sw_idx(row, p0 + pp)], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= sc;
        sm.dos[(p0 + pp) * kC + row] = pack8_bf16(f);
      }
      if (upper && wg == 1) {
        sm.dos[kPanels * kC + row] = make_uint4(pack_bf16(w * dqn, 0.f), 0, 0, 0);
        // sum_j E_tj = (don - w q.R) / den + dqn (qn - w q.n_in);  Ew_t = w (q.R / den + dqn q.n_in)
        sm.gg.rowsum[row] = fmaf(don - w * s_all, inv, dqn * (qn - w * z_all));
        sm.gg.ew[row] = w * fmaf(s_all, inv, dqn * z_all);
        float dme = p.eps * dden;
        if (it == 0 && row == valid - 1) {   // the next carry depends on m_T explicitly: dm_last - <dC_last, C_T> - <dn_last, n_T>
          float gsum = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) gsum += sm.gg.gauge[i];
          dme += (p.dm_last ? p.dm_last[bh] : 0.f) - gsum;
        }
        sm.gg.dmexp[row] = dme;
      }
      // Ek_j = kappa_j [v_j | 1] . Y_j: the two lower threads of token row j split Y's 72 columns 40 / 32 (the
      // tensor-memory loads are warp-wide; the upper lanes discard theirs)
      {
        float y[40];
        if (wg == 0) tmem_ld_row<40>(lane_base + kColY, y);
        else tmem_ld_row<32>(lane_base + kColY + 40, y);
        if (!upper) {
          float acc = 0.f;
          if (wg == 0) {
#pragma unroll
            for (int pn = 0; pn < 5; ++pn) {
              float f[8];
              unpack8_bf16(sm.v[sw_idx(row, pn)], f);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc = fmaf(f[e], y[pn * 8 + e], acc);
            }
          } else {
#pragma unroll
            for (int pn = 0; pn < 3; ++pn) {
              float f[8];
              unpack8_bf16(sm.v[sw_idx(row, 5 + pn)], f);
#pragma unroll
              for (int e = 0; e < 8; ++e) acc = fmaf(f[e], y[pn * 8 + e], acc);
            }
            acc += (row < valid ? 1.f : 0.f) * y[24];     // the "1" column
          }
          sm.gg.ekpart[wg][row] = sm.gates.kappa[row] * acc;
        }
      }
    }
    MXK_TMB(8);
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    MXK_TMB(9);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand keep_k = sw_operand(smem_u32(sm.kk), false);
      const Operand keep_v = sw_operand(smem_u32(sm.vk), false);
      const Operand keep_vx{smem_u32(sm.vkx), kC, false};           // columns 64..79 of kappa o [V|1|0]
      const Operand g_k{smem_u32(sm.g), kD, false}, g_k4{smem_u32(sm.g) + 4 * 2 * kD * 16, kD, false};   // and G's K steps 0..3 / 4
      // dQ = dA' K + dOs [S|n]                             (lower, columns 0..63)
      gemm<kC / 16>(tmem + kColLo, Operand{smem_u32(sm.dp), kC, false}, sw_operand(smem_u32(sm.k), true), id_km, false, leader);
      gemm<5>(tmem + kColLo, Operand{smem_u32(sm.dos), kC, false}, Operand{smem_u32(sm.s), kD, false}, id_kk, true, leader);
      // dK = dA'^T Q + kappa o [V|1] [G|gn]^T              (upper, columns 0..63)
      gemm<kC / 16>(tmem + kUpper + kColLo, Operand{smem_u32(sm.dp), kC, true}, sw_operand(smem_u32(sm.q), true), id_mm, false, leader);
      gemm<4>(tmem + kUpper + kColLo, keep_v, g_k, id_kk, true, leader);
      gemm<1>(tmem + kUpper + kColLo, keep_vx, g_k4, id_kk, true, leader);
      // dV = Pn^T dH + (kappa o K) G^T                     (lower, columns 64..127)
      gemm<kC / 16>(tmem + kColHi, Operand{smem_u32(sm.pn), kC, true}, sw_operand(smem_u32(sm.d_o), true), id_mm, false, leader);
      gemm<kD / 16>(tmem + kColHi, keep_k, Operand{smem_u32(sm.g), kD, true}, id_km, true, leader);
      // [G|gn]^T = delta [G|gn]^T + Q^T dOs                (upper, columns 64..135)
      gemm<kC / 16>(tmem + kUpper + kColHi, sw_operand(smem_u32(sm.q), true), Operand{smem_u32(sm.dos), kC, true}, id_g, !has_reset, leader);
      if (leader) commit(&sm.bar[1]);
    } else if (warp == 1) {
      float ed = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ed += sm.gg.edpart[i];
      chunk_gate_grads(sm.gates, sm.gg, dm, m_in, delta * ed, carry, dli_out, dlf_out, t0, p.T, p.H, lane);
      if (c > 0) {   // the next (earlier) chunk's factors; done_flags and m_in_next already hold that chunk's
        chunk_gate_scan(sm.gates, lane_gates, done_mask_from_flags(done_flags), m_in_next, 0.f, lane, (c - 1) & 1);
        lane_gates = load_lane_gates(p.log_i, p.log_f, b, h, (c - 2) * kC, p.T, p.H, lane);
      }
    }
    mbar_wait_flag(&sm.bar[1], it & 1, timed_out);
    fence_after_sync();
    if (tid == 0 && c > 0) issue_chunk_loads(c - 1);   // in flight while the output epilogue runs
    MXK_TMB(10);

    // ---- epilogue 2: every thread owns 32 (36, 40) columns of its row ----
    {
      {
        // lower: dQ, upper: dK
        float acc[32];
        tmem_ld_row<32>(lane_base + kColLo + wg * 32, acc);
        uint4* stage = upper ? sm.dp : sm.dos;
#pragma unroll
        for (int pn = 0; pn < 4; ++pn) stage[sw_idx(row, wg * 4 + pn)] = pack8_bf16(acc + pn * 8);
      }
      // lower stores dV, upper refreshes the bf16 operand copy of G | gn
      {
        float acc[40];
        if (wg == 0) tmem_ld_row<32>(lane_base + kColHi, acc);
        else tmem_ld_row<40>(lane_base + kColHi + 32, acc);
        uint4 packed[5];
#pragma unroll
        for (int pn = 0; pn < 5; ++pn)
          if (pn < gpn) packed[pn] = pack8_bf16(acc + pn * 8);
        if (upper) {
#pragma unroll
          for (int pn = 0; pn < 5; ++pn)
            if (pn < gpn) sm.g[(gp0 + pn) * kD + row] = packed[pn];
        }
        if (!upper) {
#pragma unroll
          for (int pn = 0; pn < 4; ++pn) sm.pn[sw_idx(row, wg * 4 + pn)] = packed[pn];
        }
        if (c == 0) {
          // cotangent of the carried state, and <dC_0, C_0> + <dn_0, n_0> for dm0
          float gauge = 0.f;
          if (upper && row < hd) {
            float* out = p.dc0 ? p.dc0 + (static_cast<size_t>(bh) * hd + row) * hd : nullptr;
            const float* c0 = p.c0 ? p.c0 + (static_cast<size_t>(bh) * hd + row) * hd : nullptr;
#pragma unroll
            for (int i = 0; i < 40; ++i) {
              const int vcol = gp0 * 8 + i;
              if (i < gpn * 8) {
                if (vcol < kD) {
                  if (vcol < hd) {
                    if (out) out[vcol] = acc[i];
                    if (c0) gauge = fmaf(acc[i], c0[vcol], gauge);
                  }
                } else if (vcol == kD) {
                  if (p.dn0) p.dn0[static_cast<size_t>(bh) * hd + row] = acc[i];
                  if (p.n0) gauge = fmaf(acc[i], p.n0[static_cast<size_t>(bh) * hd + row], gauge);
                }
              }
            }
          }
#pragma unroll
          for (int off = 16; off >= 1; off >>= 1) gauge += __shfl_xor_sync(0xffffffffu, gauge, off);
          if (lane == 0) sm.gg.gauge[warp] = gauge;
        }
      }
    }
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_dq, sm.dos, t0, h, b);
      tma::store_plain_tile(&p.map_dk, sm.dp, t0, h, b);
      tma::store_plain_tile(&p.map_dv, sm.pn, t0, h, b);
      tma::commit_group();
    }
    MXK_TMB(11);
  }
  if (p.dm0 && warp == 1 && lane == 0) {
    float gsum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) gsum += sm.gg.gauge[i];
    p.dm0[bh] = carry + gsum;
  }
  if (tid == 0) tma::wait_group_all();

  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kBwdTmemCols);
}

}  // namespace
}  // namespace mxk

#ifdef MXK_TIMING
extern "C" int mxk_debug_mtcb_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_mtcb_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_mtcb_phase_cycles, 16 * sizeof(unsigned long long));
}
#endif

extern "C" {

int mxk_mlstm_bf16_bwd(const void* q, const void* k, const void* v, const float* log_i, const float* log_f,
                       const float* c0, const float* n0, const float* m0, const uint8_t* done, const void* dh,
                       const float* c_last, const float* n_last, const float* m_steps, const void* chunk_states,
                       const float* dc_last, const float* dn_last, const float* dm_last, void* dq, void* dk, void* dv,
                       float* dlog_i, float* dlog_f, float* dc0, float* dn0, float* dm0, int* status, int B, int T,
                       int H, int d, float eps, mxk_stream_t stream) {
  using namespace mxk;
  using namespace mxk::linattn;
  if (!q || !k || !v || !log_i || !log_f || !dh || !m_steps || !chunk_states || !dq || !dk || !dv || !dlog_i || !dlog_f)
    return MXK_ERR_NULL;
  if ((dc_last && !c_last) || (dn_last && !n_last)) return MXK_ERR_NULL;   // the gauge term needs the forward call's next carry
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d < 8 || d > kD || d % 8) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, dh, chunk_states, (const void*)dq, (const void*)dk, (const void*)dv})
    if (!aligned16(ptr)) return MXK_ERR_ALIGN;
  for (const void* ptr : {(const void*)log_i, (const void*)log_f, (const void*)c0, (const void*)n0, (const void*)m0, (const void*)c_last,
                          (const void*)n_last, (const void*)m_steps, (const void*)dc_last, (const void*)dn_last, (const void*)dm_last,
                          (const void*)dlog_i, (const void*)dlog_f, (const void*)dc0, (const void*)dn0, (const void*)dm0})
    if (ptr && (reinterpret_cast<uintptr_t>(ptr) & 3u)) return MXK_ERR_ALIGN;
  BwdParams prm;
  prm.log_i = log_i; prm.log_f = log_f; prm.m_steps = m_steps; prm.m0 = m0; prm.c0 = c0; prm.n0 = n0;
  prm.c_last = c_last; prm.n_last = n_last;
  prm.chunk_states = static_cast<const uint4*>(chunk_states);
  prm.done = done;
  prm.dc_last = dc_last; prm.dn_last = dn_last; prm.dm_last = dm_last;
  prm.dlog_i = dlog_i; prm.dlog_f = dlog_f; prm.dc0 = dc0; prm.dn0 = dn0; prm.dm0 = dm0;
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H;
  prm.eps = eps;
  prm.d = d;
  if (!tma::make_sw_map(&prm.map_q, q, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_v, v, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_do, dh, B, T, H, kC, d))
    return MXK_ERR_UNSUPPORTED;
  if (!tma::make_sw_map(&prm.map_dq, dq, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_dk, dk, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_dv, dv, B, T, H, kC, d))
    return MXK_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(mlstm_tc_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(BwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  mlstm_tc_bwd_kernel<<<B * H, kBwdThreads, sizeof(BwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
