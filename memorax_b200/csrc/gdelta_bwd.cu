// Gated delta rule, backward, on the sm_100a tensor cores.
//
// One CTA (256 threads) owns one (batch, head) sequence and walks its 64-token
// chunks right to left with the fp32 cotangent of the state, dS (128 x 128),
// resident in tensor memory.  S_in and U of every chunk are the forward call's residual.
// With the chunk quantities of gdelta_common.cuh (A = I + diag(beta) L, P =
// tril(G o QK^T), R = V - diag(g) K S_in^T, U = A^-1 diag(beta) R):
//   dU   = P^T dO + diag(gam) K dS^T            dR = T'^T dU  with T' = A^-1 diag(beta) from the preparation
//                                                kernel (gdelta_prep.cu): a product, no back substitution
//   dV   = dR                                    dbeta_t = (dR_t . U_t) / beta_t^2
//   dP   = tril(dO U^T)                          dL = -stril(dR U^T)
//   dQ   = (dP o G) K + diag(g) dO S_in
//   dK   = (dP o G)^T Q + (dL o G) K + (dL o G)^T K + diag(gam) U dS - diag(g) dR S_in
//   dS_in = g_last dS + (diag(g) dO)^T Q - (diag(g) dR)^T K
//   decay: E = (dP o QK^T + dL o KK^T) o G,  dg_t = do_t.(S_in q_t) - dr_t.(S_in k_t),
//          dgam_j = u_j.(dS k_j),  dg_last += <dS, S_in>;
//          dcum_t = rowsum_t(E) - colsum_t(E) + dg_t g_t - dgam_t gam_t (+ sum_j dgam_j gam_j at t = last),
//          dlog(alpha_i) = sum_{t >= i} dcum_t,  dalpha_i = done_i ? 0 : dlog(alpha_i) / alpha_i.
// Matrices with d_v on their rows are kept transposed ([v][t]) so that thread v
// owns one value column, as in the forward kernel; dQ and dK are accumulated transposed too
// ([feature][token], M = 128 products: the full tensor datapath instead of half of it).
#include "gdelta_common.cuh"
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace gdelta;

struct BwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* alpha;
  const float* beta;
  const __nv_bfloat16* d_o;
  const uint4* chunk_states;
  const uint4* tprime;                // T' of every chunk (the forward call's workspace)
  const uint8_t* done;
  const float* ds_last;
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  float* dalpha;
  float* dbeta;
  float* ds0;
  int* status;
  int B, T, H;
  int d;                              // head dimension in memory: 128, or 64 (see the forward kernel)
  CUtensorMap map_k, map_q, map_do;   // 64-token tiles as SW tiles (two 64-column blocks)
  CUtensorMap map_dq, map_dk;         // the same for the outputs
  CUtensorMap map_dv;                 // 64-token tiles row-major
  unsigned long long* phase_cycles;   // per-phase cycle counters, nullptr unless switched on
};

// Row stride of the fp32 64 x 64 matrices that threads write row by row: 68 floats keep
// rows 16-byte aligned and spread the 16-byte stores of eight rows over all banks.
constexpr int kLS = kC + 4;

struct BwdSmem {
  uint4 s[kStateVecs];      // S_in bf16          [k/8][v][8]
  uint4 ds[kStateVecs];     // dS bf16            [k/8][v][8]
  uint4 k[kPanD * kC];      // K                  SW tiles (two 64-column blocks)
  uint4 q[kPanD * kC];      // Q                  SW tiles
  uint4 d_o[kPanD * kC];    // dO, later g dO     SW tiles
  uint4 r1[kC * 16];        // dU^T -> dR^T                   [t/8][v][8]   -> dq staging (SW tiles)
  uint4 r2[kC * 16];        // -(g dR)^T                      [j/8][v][8]
  uint4 u[kPanC * kD];      // U^T                [j/8][v][8]
  uint4 ug[kPanC * kD];     // (gam U)^T
  uint4 p[kPanC * kC];      // tril(G o QK^T)     [j/8][t][8]
  float l[kC * kLS];        // T' [j/8][t][8] (first 8 KiB, by bulk copy) -> E[t][j] (row stride kLS)
  float lt[kC * kC];        // dV tile -> (dP o G), (dL o G) panels -> dk staging (SW tiles)
  ChunkDecay cd;
  // per-warp partial sums of the decay cotangents, combined in a fixed order (no floating-point atomics:
  // the results are bit-reproducible)
  float dg_a[4][kC], dg_b[4][kC], dgam_p[4][kC];
  float rowsum[kC], colsum[kC], dcum[kC];
  float dgl[8];
  uint64_t bar[3];
  uint64_t bar_load;
  uint32_t tmem;
};
static_assert(sizeof(BwdSmem) <= 227 * 1024, "backward shared memory exceeds one SM");

// Per-phase cycle counters, always compiled and switched on at run time (mxk_debug_gd_phase_cycles):
// thread 0 of every 37th CTA adds the cycles since the previous mark to phase_cycles[i].  With the
// counters off this is one never-taken branch per phase.  Those branches also split the chunk loop
// into one basic block per phase, which keeps ptxas from hoisting a later phase's loads across the
// register-heavy substitution: 234 registers and no spills against 255 plus spills without them,
// and about 10 % less time per launch.
}  // namespace
__device__ unsigned long long g_gd_phase_cycles[24];
namespace {
#define MXK_TG(i) do { if (p.phase_cycles != nullptr && tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&p.phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kUpper = 16u << 16;
constexpr uint32_t kColDS = 0, kColKK = 128, kColQK = 192, kColY = 256, kColOI = 320, kColX1 = 320, kColDR = 320,
                   kColW = 320, kColX2 = 384, kColDP = 448, kColDQ = 128, kColDK = 192, kColDelta = 384;

// Sums N (32 or 64) per-thread values over the 32 lanes of a warp; on return lane l holds
// the totals of indices (N / 32) l .. (N / 32) l + N / 32 - 1 in vals[0 .. N / 32 - 1].
template <int N>
__device__ __forceinline__ void warp_reduce(float* vals, int lane) {
#pragma unroll
  for (int off = 16, n = N; off >= 1; off >>= 1, n >>= 1) {
    const int half = n >> 1;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      if (i < half) {
        const float send = upper ? vals[i] : vals[i + half];
        const float keep = upper ? vals[i + half] : vals[i];
        vals[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    }
  }
}

// All global -> shared traffic of chunk `c` (K, Q, dO, S_in, U^T): six TMA tile
// loads and two bulk copies issued by ONE thread, completing on sm.bar_load.  The
// kernel issues them one chunk ahead, right after the last MMAs of the previous chunk
// have released the buffers, so that they overlap that chunk's last epilogue.
constexpr uint32_t kChunkLoadBytes = (3 * kPanD * kC + kResidualVecs + kAinvVecs) * 16;
__device__ __forceinline__ void issue_chunk_loads(BwdSmem& sm, const BwdParams& p, int b, int h, int c, int nchunks) {
  // earlier generic-proxy accesses to these buffers are ordered before the async-proxy writes
  fence_smem_to_async();
  tma::expect_bytes(&sm.bar_load, kChunkLoadBytes);
  const int t0 = c * kC;
  // K, Q, dO as SW tiles: two 64-column blocks of 64 x 128 bytes each
  tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, t0, h, b, 0);
  tma::load_plain_tile(sm.k + kSwBlockVecs, &p.map_k, &sm.bar_load, t0, h, b, 64);
  tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, t0, h, b, 0);
  tma::load_plain_tile(sm.q + kSwBlockVecs, &p.map_q, &sm.bar_load, t0, h, b, 64);
  tma::load_plain_tile(sm.d_o, &p.map_do, &sm.bar_load, t0, h, b, 0);
  tma::load_plain_tile(sm.d_o + kSwBlockVecs, &p.map_do, &sm.bar_load, t0, h, b, 64);
  const uint4* src = p.chunk_states + (static_cast<size_t>(b * p.H + h) * nchunks + c) * kResidualVecs;
  tma::load_bulk(sm.s, src, kStateVecs * 16, &sm.bar_load);
  tma::load_bulk(sm.u, src + kStateVecs, kUVecs * 16, &sm.bar_load);
  const uint4* tp_src = p.tprime + (static_cast<size_t>(b * p.H + h) * nchunks + c) * kAinvVecs;
  tma::load_bulk(sm.l, tp_src, kAinvVecs * 16, &sm.bar_load);
  if (c > 0) {   // the chunk after it (walking right to left): into L2 now, so that its loads hit there
    const int tp = t0 - kC;
    tma::prefetch_plain_tile(&p.map_k, tp, h, b, 0);
    tma::prefetch_plain_tile(&p.map_q, tp, h, b, 0);
    tma::prefetch_plain_tile(&p.map_do, tp, h, b, 0);
    if (p.d > 64) {
      tma::prefetch_plain_tile(&p.map_k, tp, h, b, 64);
      tma::prefetch_plain_tile(&p.map_q, tp, h, b, 64);
      tma::prefetch_plain_tile(&p.map_do, tp, h, b, 64);
    }
    tma::prefetch_bulk(src - kResidualVecs, kResidualVecs * 16);
    tma::prefetch_bulk(tp_src - kAinvVecs, kAinvVecs * 16);
  }
}

// 256 threads: two warpgroups that see the same TMEM lanes (warp w and warp w + 4 share a lane
// quarter) and split every epilogue between them -- by key / state columns where a thread
// owns a token or value row, by role around the back substitution.
constexpr int kBwdThreads = 256;

__global__ void __launch_bounds__(kBwdThreads) gdelta_bwd_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;            // warpgroup
  const int qw = warp & 3;             // TMEM lane quarter of this warp
  const int vt = tid & 127;            // value row owned in the transposed (M = 128) accumulators
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int row = qw * 16 + (lane & 15);   // token row owned in the M = 64 accumulators
  const bool upper = lane >= 16;
  const int nchunks = (p.T + kC - 1) / kC;

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init(&sm.bar[2], 1);
    mbar_init(&sm.bar_load, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(qw * 32) << 16);

  const size_t bt_base = static_cast<size_t>(b) * p.T;
  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  bool timed_out = false;

  if (tid == 0) issue_chunk_loads(sm, p, b, h, nchunks - 1, nchunks);
  float2 ab_next = fetch_chunk_decay(p.alpha, p.beta, bt_base, p.H, h, (nchunks - 1) * kC, p.T, tid);
  linattn::DoneFlags flags_next = linattn::load_done_flags(drow, (nchunks - 1) * kC, p.T, lane);
  // cotangent of the next carry: thread (v, wg) owns dS[v][64 wg .. 64 wg + 63]
  {
    const float* g0 = (p.ds_last && vt < p.d && wg * 64 < p.d) ? p.ds_last + (static_cast<size_t>(bh) * p.d + vt) * p.d + wg * 64 : nullptr;
    float vals[64];   // all loads first: the TMEM stores below are compiler memory barriers
#pragma unroll
    for (int c4 = 0; c4 < 16; ++c4) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (g0) x = *reinterpret_cast<const float4*>(g0 + c4 * 4);
      vals[c4 * 4] = x.x; vals[c4 * 4 + 1] = x.y; vals[c4 * 4 + 2] = x.z; vals[c4 * 4 + 3] = x.w;
    }
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
      tmem_st8(lane_base + kColDS + wg * 64 + c8 * 8, vals + c8 * 8);
      sm.ds[(wg * 8 + c8) * kD + vt] = pack8_bf16(vals + c8 * 8);
    }
    tmem_st_wait();
  }

  long long t_prev_ = clock64();

  for (int it = 0; it < nchunks; ++it) {
    const int c = nchunks - 1 - it;
    const int t0 = c * kC;
    const int valid = min(kC, p.T - t0);
    const uint64_t dm = linattn::done_mask_from_flags(flags_next);
    __syncthreads();
    chunk_decay_from_regs(sm.cd, ab_next, dm, tid);
    if (tid < kC) sm.rowsum[tid] = 0.f;   // two contributions per row: order-independent

    MXK_TG(0);
    mbar_wait_flag(&sm.bar_load, it & 1, timed_out);
    // (gam U)^T from row v of U^T, four panels per warpgroup
#pragma unroll
    for (int j4 = 0; j4 < kPanC / 2; ++j4) {
      const int jp = wg * (kPanC / 2) + j4;
      float f[8];
      unpack8_bf16(sm.u[jp * kD + vt], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= sm.cd.gam[jp * 8 + e];
      sm.ug[jp * kD + vt] = pack8_bf16(f);
    }
    if (tid == 0) tma::wait_group_read<0>();   // the previous chunk's dq / dk tiles have left `r1` / `lt`
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    MXK_TG(1);
    // ---- MMAs A: K K^T, Q K^T, Y^T = S_in K^T, OI^T = S_in Q^T, X2^T = dS K^T ----
    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      constexpr uint32_t kBlk = kSwBlockVecs * 16;   // bytes between the two 64-column blocks of an SW tile pair
      const Operand ak = sw_operand(smem_u32(sm.k), false, kBlk), aq = sw_operand(smem_u32(sm.q), false, kBlk);
      const Operand as{smem_u32(sm.s), kD, false}, ads{smem_u32(sm.ds), kD, false};
      const uint32_t id_128 = idesc_bf16(kD, kC, false, false);
      // 64 x 64 products are issued as two N = 32 halves: keys 0..31 land in lanes 0..15 of each
      // warp's TMEM quarter, keys 32..63 in lanes 16..31 of the same columns, so both half-warps
      // work on the same token row in the epilogues
      const Operand bk_lo = ak, bk_hi = sw_operand(smem_u32(sm.k) + 32 * 128, false, kBlk);
      const uint32_t id_half = idesc_bf16(kC, 32, false, false);
      gemm128(tmem + kColKK, ak, bk_lo, id_half, false, leader);
      gemm128(tmem + kUpper + kColKK, ak, bk_hi, id_half, false, leader);
      gemm128(tmem + kColQK, aq, bk_lo, id_half, false, leader);
      gemm128(tmem + kUpper + kColQK, aq, bk_hi, id_half, false, leader);
      gemm128(tmem + kColY, as, ak, id_128, false, leader);
      gemm128(tmem + kColOI, as, aq, id_128, false, leader);
      gemm128(tmem + kColX2, ads, ak, id_128, false, leader);
      if (leader) commit(&sm.bar[0]);
    }
    mbar_wait_flag(&sm.bar[0], 0, timed_out);
    fence_after_sync();
    MXK_TG(2);

    // ---- epilogue A1: tril(G o QK^T) (bf16); every thread owns 16 keys of its token row ----
    {
      const int lo = row_first_key(dm, row);
      const float cum_t = sm.cd.cum[row];
      const int j0 = (upper ? 32 : 0) + wg * 16;
      float qk[16];
      tmem_ld_row<16>(lane_base + kColQK + wg * 16, qk);
#pragma unroll
      for (int jq = 0; jq < 2; ++jq) {
        float pm[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int x = jq * 8 + e, j = j0 + x;
          const bool in = (j >= lo && j <= row);
          pm[e] = in ? __expf(cum_t - sm.cd.cum[j]) * qk[x] : 0.f;
        }
        sm.p[((j0 >> 3) + jq) * kC + row] = pack8_bf16(pm);
      }
    }
    // ---- epilogue A2: first dg term, dg_t += sum_v dO[t][v] (S_in q_t)[v]; thread (v, wg) covers
    //      tokens 32 wg .. 32 wg + 31 ----
    {
      float r[32];
      tmem_ld_row<32>(lane_base + kColOI + wg * 32, r);
#pragma unroll
      for (int t = 0; t < 32; ++t) r[t] *= sw_bf16_at(sm.d_o, wg * 32 + t, vt);
      warp_reduce<32>(r, lane);
      sm.dg_a[qw][wg * 32 + lane] = r[0];
    }
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    MXK_TG(3);
    // ---- MMAs B: X1^T = dO^T P (128 x 64), DP = dO U^T (64 x 64) ----
    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      constexpr uint32_t kBlk = kSwBlockVecs * 16;
      gemm<kC / 16>(tmem + kColX1, sw_operand(smem_u32(sm.d_o), true, kBlk), Operand{smem_u32(sm.p), kC, true}, idesc_bf16(kD, kC, true, true), false, leader);
      gemm128(tmem + kColDP, sw_operand(smem_u32(sm.d_o), false, kBlk), Operand{smem_u32(sm.u), kD, true}, idesc_bf16(kC, 32, false, true), false, leader);
      gemm128(tmem + kUpper + kColDP, sw_operand(smem_u32(sm.d_o), false, kBlk), Operand{smem_u32(sm.u) + 4 * kD * 16, kD, true}, idesc_bf16(kC, 32, false, true), false, leader);
      if (leader) commit(&sm.bar[1]);
    }
    mbar_wait_flag(&sm.bar[1], 0, timed_out);
    fence_after_sync();
    MXK_TG(4);

    // ---- epilogue B1: dU^T = X1^T + gam o X2^T as the bf16 operand of the T' product, and the dgam
    //      reduction dgam_j = sum_v u_j[v] (dS k_j)[v]; thread (v, wg) covers tokens 32 wg .. 32 wg + 31 ----
    {
      float x2[32], x1[32];
      tmem_ld_row<32>(lane_base + kColX2 + wg * 32, x2);   // (dS k_j)[v]
      tmem_ld_row<32>(lane_base + kColX1 + wg * 32, x1);
#pragma unroll
      for (int tp = 0; tp < 4; ++tp) {
        float du[8], uf[8];
        unpack8_bf16(sm.u[(wg * 4 + tp) * kD + vt], uf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int t = tp * 8 + e;
          du[e] = fmaf(sm.cd.gam[wg * 32 + t], x2[t], x1[t]);
          x2[t] *= uf[e];
        }
        sm.r1[(wg * 4 + tp) * kD + vt] = pack8_bf16(du);
      }
      warp_reduce<32>(x2, lane);
      sm.dgam_p[qw][wg * 32 + lane] = x2[0];
    }
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    MXK_TG(11);
    // ---- MMA B2: dR^T = dU^T T'  (128 x 64, contraction over the 64 tokens of dU) ----
    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      gemm<kC / 16>(tmem + kColDR, Operand{smem_u32(sm.r1), kD, false}, Operand{smem_u32(sm.l), kC, true},
                    idesc_bf16(kD, kC, false, true), false, leader);
      if (leader) commit(&sm.bar[2]);
    }
    // meanwhile: <dS, S_in> for the g_last gradient; thread (v, wg) covers state columns 64 wg .. 64 wg + 63
    {
      float dot = 0.f;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        const int q4 = wg * 2 + q2;
        float d32[32];
        tmem_ld_row<32>(lane_base + kColDS + q4 * 32, d32);
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float s8[8];
          unpack8_bf16(sm.s[(q4 * 4 + c8) * kD + vt], s8);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(d32[c8 * 8 + e], s8[e], dot);
        }
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      if (lane == 0) sm.dgl[warp] = dot;
    }
    mbar_wait_flag(&sm.bar[2], it & 1, timed_out);
    fence_after_sync();
    MXK_TG(12);

    // ---- epilogue B2: dR = dV: the dV tile (row-major [t][v], staged in `lt`), -(g dR)^T and dR^T
    //      panels, and dg_t -= dr_t . (S_in k_t) ----
    {
      float dr[32], y[32];
      tmem_ld_row<32>(lane_base + kColDR + wg * 32, dr);
      tmem_ld_row<32>(lane_base + kColY + wg * 32, y);
      __nv_bfloat16* dvt = reinterpret_cast<__nv_bfloat16*>(sm.lt);
#pragma unroll
      for (int tp = 0; tp < 4; ++tp) {
        float ng[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int t = tp * 8 + e;
          dvt[(wg * 32 + t) * kD + vt] = __float2bfloat16(dr[t]);
          ng[e] = -sm.cd.g[wg * 32 + t] * dr[t];
          y[t] *= -dr[t];
        }
        sm.r1[(wg * 4 + tp) * kD + vt] = pack8_bf16(dr + tp * 8);
        sm.r2[(wg * 4 + tp) * kD + vt] = pack8_bf16(ng);
      }
      MXK_TG(13);
      warp_reduce<32>(y, lane);
      sm.dg_b[qw][wg * 32 + lane] = y[0];
      MXK_TG(14);
    }
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    if (tid == 0) {   // the dV tile leaves by one TMA store (rows past the end of the sequence are clipped)
      tma::store_plain_tile(&p.map_dv, sm.lt, t0, h, b);
      tma::commit_group();
    }

    MXK_TG(5);
    // ---- MMA C: W' = dR U^T (64 x 64) ----
    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      gemm<kD / 16>(tmem + kColW, Operand{smem_u32(sm.r1), kD, true}, Operand{smem_u32(sm.u), kD, true}, idesc_bf16(kC, 32, true, true), false, leader);
      gemm<kD / 16>(tmem + kUpper + kColW, Operand{smem_u32(sm.r1), kD, true}, Operand{smem_u32(sm.u) + 4 * kD * 16, kD, true}, idesc_bf16(kC, 32, true, true), false, leader);
      if (leader) commit(&sm.bar[0]);
    }
    mbar_wait_flag(&sm.bar[0], 1, timed_out);
    fence_after_sync();
    MXK_TG(6);
    if (tid == 0) tma::wait_group_read<0>();   // the dV tile has left `lt` before it is reused
    __syncthreads();
    MXK_TG(15);

    // ---- epilogue C: (dP o G), (dL o G), E, dbeta; g-scaled dO.  Every thread owns 16 keys of
    //      its token row ----
    {
      uint4* dpg = reinterpret_cast<uint4*>(sm.lt);           // [j/8][t][8]
      uint4* dlg = dpg + kPanC * kC;
      const int lo = row_first_key(dm, row);
      const float cum_t = sm.cd.cum[row], beta_t = sm.cd.beta[row];
      const int j0 = (upper ? 32 : 0) + wg * 16;
      float rs = 0.f, wtt = 0.f;
      float kk[16], qk[16], dp[16], w[16];
      tmem_ld_row<16>(lane_base + kColKK + wg * 16, kk);
      tmem_ld_row<16>(lane_base + kColQK + wg * 16, qk);
      tmem_ld_row<16>(lane_base + kColDP + wg * 16, dp);
      tmem_ld_row<16>(lane_base + kColW + wg * 16, w);
      MXK_TG(16);
#pragma unroll
      for (int jq = 0; jq < 2; ++jq) {
        float a8[8], b8[8], ev[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int x = jq * 8 + e, j = j0 + x;
          const bool in = (j >= lo && j <= row);
          const float gtj = in ? __expf(cum_t - sm.cd.cum[j]) : 0.f;
          const float dl = (j < row) ? -w[x] : 0.f;
          wtt = (j == row) ? w[x] : wtt;   // the diagonal of W', held by exactly one thread per row
          a8[e] = dp[x] * gtj;
          b8[e] = dl * gtj;
          ev[e] = (dp[x] * qk[x] + dl * kk[x]) * gtj;
          rs += ev[e];
        }
        float4* erow = reinterpret_cast<float4*>(&sm.l[row * kLS + j0 + jq * 8]);
        erow[0] = make_float4(ev[0], ev[1], ev[2], ev[3]);
        erow[1] = make_float4(ev[4], ev[5], ev[6], ev[7]);
        const int pn = (j0 >> 3) + jq;
        dpg[pn * kC + row] = pack8_bf16(a8);
        dlg[pn * kC + row] = pack8_bf16(b8);
      }
      MXK_TG(17);
      // dbeta_t = (dR_t . U_t) / beta_t^2, once, outside the unrolled loop (a store inside it made every
      // iteration a divergent branch for the warps that hold the diagonal)
      if (row >= j0 && row < j0 + 16 && row < valid)
        p.dbeta[(static_cast<size_t>(b) * p.T + t0 + row) * p.H + h] = beta_t != 0.f ? wtt / (beta_t * beta_t) : 0.f;
      rs += __shfl_xor_sync(0xffffffffu, rs, 16);
      if (!upper) atomicAdd(&sm.rowsum[row], rs);
      const float gt = sm.cd.g[row];
      const int p0 = (upper ? kPanD / 2 : 0) + wg * (kPanD / 4);
#pragma unroll
      for (int pp = 0; pp < kPanD / 4; ++pp) {
        float f[8];
        unpack8_bf16(sm.d_o[sw_slot(row, p0 + pp)], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= gt;
        sm.d_o[sw_slot(row, p0 + pp)] = pack8_bf16(f);
      }
    }
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    MXK_TG(7);
    // ---- MMAs D: dQ^T, dK^T (128 x 64 each: features on the rows), dS_in increment (128 x 128) ----
    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const uint4* dpg_p = reinterpret_cast<const uint4*>(sm.lt);
      const uint32_t dpg = smem_u32(dpg_p), dlg = smem_u32(dpg_p + kPanC * kC);
      constexpr uint32_t kBlk = kSwBlockVecs * 16;
      const Operand kt = sw_operand(smem_u32(sm.k), true, kBlk), qt = sw_operand(smem_u32(sm.q), true, kBlk);   // K^T, Q^T
      const Operand bk = kt, bq = qt;
      const Operand gdo_k = sw_operand(smem_u32(sm.d_o), false, kBlk), gdo_t = sw_operand(smem_u32(sm.d_o), true, kBlk);
      const Operand st{smem_u32(sm.s), kD, true}, dst{smem_u32(sm.ds), kD, true};                               // S_in^T, dS^T
      const uint32_t id_mk = idesc_bf16(kD, kC, true, false), id_mm64 = idesc_bf16(kD, kC, true, true);
      // dQ^T = K^T (dP o G)^T + S_in^T (g dO)^T
      gemm<kC / 16>(tmem + kColDQ, kt, Operand{dpg, kC, false}, id_mk, false, leader);
      gemm128(tmem + kColDQ, st, gdo_k, id_mk, true, leader);
      // dK^T = Q^T (dP o G) + K^T (dL o G)^T + K^T (dL o G) + dS^T (gam U)^T - S_in^T (g dR)^T
      gemm<kC / 16>(tmem + kColDK, qt, Operand{dpg, kC, true}, id_mm64, false, leader);
      gemm<kC / 16>(tmem + kColDK, kt, Operand{dlg, kC, false}, id_mk, true, leader);
      gemm<kC / 16>(tmem + kColDK, kt, Operand{dlg, kC, true}, id_mm64, true, leader);
      gemm<kD / 16>(tmem + kColDK, dst, Operand{smem_u32(sm.ug), kD, true}, id_mm64, true, leader);
      gemm<kD / 16>(tmem + kColDK, st, Operand{smem_u32(sm.r2), kD, true}, id_mm64, true, leader);
      // dS_in - g_last dS = (g dO)^T Q - (g dR)^T K
      gemm<kC / 16>(tmem + kColDelta, gdo_t, bq, idesc_bf16(kD, kD, true, true), false, leader);
      gemm<kC / 16>(tmem + kColDelta, Operand{smem_u32(sm.r2), kD, false}, bk, idesc_bf16(kD, kD, false, true), true, leader);
      if (leader) commit(&sm.bar[1]);
    }

    // ---- decay gradients, by warps 2..3 / warp 2 while warp 0 is issuing the MMAs above ----
    if (tid >= 64 && tid < 128) {
      const int x = tid - 64;
      float cs = 0.f;
#pragma unroll 8
      for (int t = 0; t < kC; ++t) cs += sm.l[t * kLS + x];
      asm volatile("bar.arrive 3, 96;" ::: "memory");   // E has been read: warp 0 may let the next T' land over it
      const float dg = ((sm.dg_a[0][x] + sm.dg_a[1][x]) + (sm.dg_a[2][x] + sm.dg_a[3][x])) +
                       ((sm.dg_b[0][x] + sm.dg_b[1][x]) + (sm.dg_b[2][x] + sm.dg_b[3][x]));
      const float dgam = (sm.dgam_p[0][x] + sm.dgam_p[1][x]) + (sm.dgam_p[2][x] + sm.dgam_p[3][x]);
      sm.dcum[x] = sm.rowsum[x] - cs + dg * sm.cd.g[x] - dgam * sm.cd.gam[x];
      sm.colsum[x] = dgam * sm.cd.gam[x];
      asm volatile("bar.sync 2, 64;" ::: "memory");   // warps 2 and 3 only
      if (x < 32) {
        float extra = sm.colsum[2 * x] + sm.colsum[2 * x + 1];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) extra += __shfl_xor_sync(0xffffffffu, extra, off);
        extra += (((sm.dgl[0] + sm.dgl[1]) + (sm.dgl[2] + sm.dgl[3])) + ((sm.dgl[4] + sm.dgl[5]) + (sm.dgl[6] + sm.dgl[7]))) * sm.cd.g[kC - 1];
        float d0 = sm.dcum[2 * x], d1 = sm.dcum[2 * x + 1];
        if (x == 31) d1 += extra;
        // suffix sums over the chunk
        float s = d0 + d1;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const float o = __shfl_down_sync(0xffffffffu, s, off);
          if (x + off < 32) s += o;
        }
        const float dla0 = s, dla1 = s - d0;
        const size_t base = (static_cast<size_t>(b) * p.T + t0) * p.H + h;
        const int i0 = 2 * x, i1 = 2 * x + 1;
        if (i0 < valid) p.dalpha[base + static_cast<size_t>(i0) * p.H] = ((dm >> i0) & 1ull) ? 0.f : dla0 / sm.cd.alpha[i0];
        if (i1 < valid) p.dalpha[base + static_cast<size_t>(i1) * p.H] = ((dm >> i1) & 1ull) ? 0.f : dla1 / sm.cd.alpha[i1];
      }
    }

    MXK_TG(8);
    mbar_wait_flag(&sm.bar[1], 1, timed_out);
    fence_after_sync();
    MXK_TG(9);
    // the MMAs above were the last readers of the staged tiles: fetch the next chunk (its T' lands over E, which
    // warps 2..3 have finished reading once they have arrived on barrier 3)
    if (warp == 0) asm volatile("bar.sync 3, 96;" ::: "memory");
    if (c > 0) {
      if (tid == 0) issue_chunk_loads(sm, p, b, h, c - 1, nchunks);
      ab_next = fetch_chunk_decay(p.alpha, p.beta, bt_base, p.H, h, t0 - kC, p.T, tid);
      flags_next = linattn::load_done_flags(drow, t0 - kC, p.T, lane);
    }

    // ---- epilogue D: dq, dk tiles from the transposed accumulators (thread (feature, wg) covers tokens
    //      32 wg .. 32 wg + 31); dS = g_last dS + increment, 64 state columns per warpgroup ----
    {
      // staged as SW tiles in buffers the finished MMAs no longer need (dq in `r1`, dk in `lt`),
      // stored by TMA after the barrier that ends the chunk
      uint4* dq_stage = sm.r1;
      uint4* dk_stage = reinterpret_cast<uint4*>(sm.lt);
      {
        float acc[32];
        tmem_ld_row<32>(lane_base + kColDQ + wg * 32, acc);
#pragma unroll
        for (int e = 0; e < 32; ++e)
          reinterpret_cast<__nv_bfloat16*>(&dq_stage[sw_slot(wg * 32 + e, vt >> 3)])[vt & 7] = __float2bfloat16(acc[e]);
        tmem_ld_row<32>(lane_base + kColDK + wg * 32, acc);
#pragma unroll
        for (int e = 0; e < 32; ++e)
          reinterpret_cast<__nv_bfloat16*>(&dk_stage[sw_slot(wg * 32 + e, vt >> 3)])[vt & 7] = __float2bfloat16(acc[e]);
      }
      const float g_last = sm.cd.g[kC - 1];
      float* out0 = (c == 0 && p.ds0 && vt < p.d) ? p.ds0 + (static_cast<size_t>(bh) * p.d + vt) * p.d : nullptr;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        const int q4 = wg * 2 + q2;
        float s[32], inc[32];
        tmem_ld_row<32>(lane_base + kColDS + q4 * 32, s);
        tmem_ld_row<32>(lane_base + kColDelta + q4 * 32, inc);
#pragma unroll
        for (int e = 0; e < 32; ++e) s[e] = fmaf(g_last, s[e], inc[e]);
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          tmem_st8(lane_base + kColDS + q4 * 32 + c8 * 8, s + c8 * 8);
          sm.ds[(q4 * 4 + c8) * kD + vt] = pack8_bf16(s + c8 * 8);
          if (out0 && q4 * 32 < p.d) {
            *reinterpret_cast<float4*>(out0 + q4 * 32 + c8 * 8) = make_float4(s[c8 * 8], s[c8 * 8 + 1], s[c8 * 8 + 2], s[c8 * 8 + 3]);
            *reinterpret_cast<float4*>(out0 + q4 * 32 + c8 * 8 + 4) = make_float4(s[c8 * 8 + 4], s[c8 * 8 + 5], s[c8 * 8 + 6], s[c8 * 8 + 7]);
          }
        }
      }
      tmem_st_wait();
    }
    MXK_TG(10);
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_dq, sm.r1, t0, h, b, 0);
      tma::store_plain_tile(&p.map_dk, sm.lt, t0, h, b, 0);
      if (p.d > 64) {   // a 64-wide head has no second column block in memory
        tma::store_plain_tile(&p.map_dq, sm.r1 + kSwBlockVecs, t0, h, b, 64);
        tma::store_plain_tile(&p.map_dk, reinterpret_cast<uint4*>(sm.lt) + kSwBlockVecs, t0, h, b, 64);
      }
      tma::commit_group();
    }
  }
  if (tid == 0) tma::wait_group_all();

  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace mxk

namespace mxk {
namespace {
bool g_gd_phase_on = false;
}  // namespace
}  // namespace mxk

// Debug hook (not part of the C ABI in mxk.h): reset > 0 zeroes the 24 phase counters and switches them
// on for later launches, reset < 0 switches them off, reset == 0 copies them to `out`.
extern "C" int mxk_debug_gd_phase_cycles(unsigned long long* out, int reset) {
  if (reset != 0) {
    mxk::g_gd_phase_on = reset > 0;
    unsigned long long z[24] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_gd_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_gd_phase_cycles, 24 * sizeof(unsigned long long));
}

extern "C" {

int mxk_gdelta_bf16_bwd(const void* q, const void* k, const void* v, const float* alpha, const float* beta,
                        const void* d_o, const void* chunk_states, const void* workspace, const uint8_t* done,
                        const float* ds_last,
                        void* dq, void* dk, void* dv, float* dalpha, float* dbeta, float* ds0, int* status,
                        int B, int T, int H, int d, mxk_stream_t stream) {
  using namespace mxk;
  using namespace mxk::gdelta;
  if (!q || !k || !v || !alpha || !beta || !d_o || !chunk_states || !workspace || !dq || !dk || !dv || !dalpha || !dbeta)
    return MXK_ERR_NULL;
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d != kD && d != 64) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, d_o, chunk_states, workspace, (const void*)dq, (const void*)dk, (const void*)dv,
                          (const void*)ds_last, (const void*)ds0})
    if (ptr && !aligned16(ptr)) return MXK_ERR_ALIGN;
  BwdParams prm;
  prm.q = static_cast<const __nv_bfloat16*>(q);
  prm.k = static_cast<const __nv_bfloat16*>(k);
  prm.v = static_cast<const __nv_bfloat16*>(v);
  prm.alpha = alpha;
  prm.beta = beta;
  prm.d_o = static_cast<const __nv_bfloat16*>(d_o);
  prm.chunk_states = static_cast<const uint4*>(chunk_states);
  prm.tprime = static_cast<const uint4*>(workspace);
  prm.done = done;
  prm.ds_last = ds_last;
  prm.dq = static_cast<__nv_bfloat16*>(dq);
  prm.dk = static_cast<__nv_bfloat16*>(dk);
  prm.dv = static_cast<__nv_bfloat16*>(dv);
  prm.dalpha = dalpha;
  prm.dbeta = dbeta;
  prm.ds0 = ds0;
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H; prm.d = d;
  prm.phase_cycles = nullptr;
  if (g_gd_phase_on) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_gd_phase_cycles) == cudaSuccess) prm.phase_cycles = static_cast<unsigned long long*>(sym);
  }
  if (!tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_q, q, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_do, d_o, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_dq, dq, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_dk, dk, B, T, H, kC, d) || !tma::make_plain_map(&prm.map_dv, dv, B, T, H, d, kC, kD))
    return MXK_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(gdelta_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(BwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  gdelta_bwd_kernel<<<B * H, kBwdThreads, sizeof(BwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
