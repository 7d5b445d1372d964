// Backward of chunked causal linear attention on the sm_100a tensor cores.
//
// One CTA (256 threads, two warpgroups) owns one (batch, head) sequence and walks
// its 64-token chunks right to left, carrying G^T = (dL/dS)^T with gz = dL/dz as one extra column in
// tensor memory (fp32).  The state entering each chunk comes from the forward
// call's residual (bf16, already in operand order).  Per chunk, with
// D_i = max(den_i, eps), c_i = [den_i > eps]:
//   phase 1 (independent MMAs):  P = phi(Q) phi(K)^T,  dA = dO V^T,  R = dO S_in
//   epilogue 1 (four threads per query row, 16 keys each):
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
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace linattn;

constexpr int kPanelsK = kPanels + 2;  // 80 columns: a K = 80 contraction needs whole K=16 steps
// kWgs warpgroups that see the same TMEM lanes (warps w, w + 4, ... share a lane quarter) and
// split the columns of every row between them.  Two is the measured optimum: four (512 threads, 60
// registers, no spills) gave the same results 7 % slower on the 256 x 4 x 256 x 64 workload -- the
// chunk time is the chain of barriers and of the MMA-issuing warp, not the threads' column work.
#ifndef MXK_LINATTN_BWD_THREADS
#define MXK_LINATTN_BWD_THREADS 256
#endif
constexpr int kBwdThreads = MXK_LINATTN_BWD_THREADS;
constexpr int kWgs = kBwdThreads / 128;
static_assert(kWgs == 2 || kWgs == 4, "two or four warpgroups");
constexpr int kKeysPerThread = 32 / kWgs;        // keys / state features of a query row per thread in epilogue 1
constexpr int kColsPerThread = 64 / kWgs;        // dphiQ / dphiK columns per thread in epilogue 2
constexpr int kGPanels = 8 / kWgs;               // panels of the 72-column G | gz accumulator per warpgroup
constexpr int kGPanelsMax = kGPanels + 1;        // the last warpgroup also takes the gz panel

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
  int d;   // head dimension: a multiple of 8, at most kD; the tiles are kD wide, the rest zero
  CUtensorMap map_q, map_k, map_v, map_do;   // 64-token tiles as SW tiles
  CUtensorMap map_dq, map_dk, map_dv;        // the same for the outputs
};

struct BwdSmem {
  // 128-byte-swizzled row-major tiles (umma.cuh "SW tiles"), 8 KB each, 1024-byte aligned
  uint4 q[kPanels * kC];      // phi(Q)
  uint4 k[kPanels * kC];      // phi(K)
  uint4 v[kPanels * kC];      // V
  uint4 d_o[kPanels * kC];    // dO
  uint4 kk[kPanels * kC];     // keep rows of phi(K)    (written only for chunks with a reset)
  uint4 vk[kPanels * kC];     // keep rows of V         (written only for chunks with a reset)
  // panel format
  uint4 vx[2 * kC];           // columns 64..79 of V | 1 | 0: the "1" column of the valid rows, then zeros
  uint4 vkx[2 * kC];          // the same for the keep rows
  uint4 dos[kPanelsK * kC];   // live rows of dO/D | dden | 0
  uint4 s[kPanelsK * kD];     // S_in^T | z_in | 0      [v/8][k]
  uint4 g[kPanelsK * kD];     // G^T | gz | 0           [v/8][k]
  uint4 pn[kPanels * kC];     // P / D                  [j/8][i]
  uint4 dp[kPanels * kC];     // dP                     [j/8][i]
  float xch[kWgs][2][kC];     // per warpgroup: partial den and don of every query row
  uint64_t bar[2];
  uint64_t bar_load;
  uint64_t bar_free;   // every thread arrives once it has taken its phi(Q) / phi(K) vectors for the epilogue
  uint32_t tmem;
};
static_assert(sizeof(BwdSmem) <= 113 * 1024, "two CTAs per SM");

// 256 TMEM columns per CTA (two CTAs per SM).  M = 64 accumulators use 16 of a
// warp's 32 TMEM lanes, so lanes 0..15 ("lower" threads) and 16..31 ("upper"
// threads) hold different matrices in the same columns:
//   columns   0.. 63   first P (0..31) and dA (32..63), each issued as two N = 32 halves: keys
//                      0..31 in the lower lanes, keys 32..63 in the upper lanes, so that both
//                      half-warps own 32 keys of the same query row; later dphiQ (lower) and
//                      dphiK (upper)
//   columns  64..135   lower: dV                  upper: G^T | gz (persistent)
//   columns 136..167   R, state features 0..31 in the lower lanes, 32..63 in the upper lanes
// Within a half-warp's 32 columns, warpgroup 0 takes the first 16 and warpgroup 1 the rest.
#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_bwd_phase_cycles[16];
namespace {
#define MXK_TB(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_bwd_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_TB(i) do {} while (0)
#endif
constexpr uint32_t kBwdTmemCols = 256;
#ifndef MXK_LINATTN_AHEAD
#define MXK_LINATTN_AHEAD 1
#endif
// Chunks whose tiles are requested into L2 ahead of their load.  One is the measured optimum at four chunks per
// sequence: requesting a whole sequence at its start (4) puts the first tiles behind the prefetch traffic of all
// resident CTAs and measured 7 % slower.
constexpr int kAhead = MXK_LINATTN_AHEAD;
constexpr uint32_t kUpper = 16u << 16;
constexpr uint32_t kColLo = 0, kColHi = 64, kColP = 0, kColA = 32, kColR = 136;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }

// kFull: head dimension = the tile width (compile-time bounds); otherwise a multiple of 8 below it.
template <bool kFull>
__global__ void __launch_bounds__(kBwdThreads, 2) linattn_bwd_kernel(const __grid_constant__ BwdParams p) {
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
  const int hd = kFull ? kD : p.d;   // head dimension
  const int dpan = hd >> 3;

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_free, kBwdThreads);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kBwdTmemCols);
  // zero padding panels that never change (columns 72..79 of the 80-wide operands)
  if (tid < kC) {
    sm.vx[kC + tid] = zero4;
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

  // A chunk's tiles arrive by TMA as SW tiles (S_in, the forward call's residual, by bulk copy), issued
  // by one thread the moment the previous chunk's second MMA group has completed.  The epilogue still
  // needs phi(Q) / phi(K) for the feature-map derivative, so every thread copies its four vectors into
  // registers while the MMAs run and arrives on bar_free; the issuing thread waits for that barrier.
  auto prefetch_chunk = [&](int cc) {
    tma::prefetch_plain_tile(&p.map_q, cc * kC, h, b);
    tma::prefetch_plain_tile(&p.map_k, cc * kC, h, b);
    tma::prefetch_plain_tile(&p.map_v, cc * kC, h, b);
    tma::prefetch_plain_tile(&p.map_do, cc * kC, h, b);
    tma::prefetch_bulk(p.chunk_states + (static_cast<size_t>(bh) * nchunks + cc) * (kPanelsX * kD), kPanelsX * kD * 16);
  };
  auto issue_chunk_loads = [&](int cc) {
    fence_smem_to_async();   // earlier generic-proxy accesses to the buffers come first
    tma::expect_bytes(&sm.bar_load, (4 * kPanels * kC + kPanelsX * kD) * 16);
    tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.v, &p.map_v, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.d_o, &p.map_do, &sm.bar_load, cc * kC, h, b);
    tma::load_bulk(sm.s, p.chunk_states + (static_cast<size_t>(bh) * nchunks + cc) * (kPanelsX * kD),
                   kPanelsX * kD * 16, &sm.bar_load);
    // a chunk kAhead positions on (walking right to left): into L2 now, so that its loads hit there
    if (cc - kAhead >= 0) prefetch_chunk(cc - kAhead);
  };
  if (tid == 0) {
    issue_chunk_loads(nchunks - 1);
    for (int a = 1; a < kAhead && nchunks - 1 - a >= 0; ++a) prefetch_chunk(nchunks - 1 - a);
  }

  // Cotangent of the next carry -> TMEM (upper lanes) and its bf16 operand copy
  // (upper thread `row` owns G^T[row][.] = dS[.][row]; warpgroup 0 takes value columns
  // 0..31, warpgroup 1 columns 32..63 and gz).
  const int gp0 = wg * kGPanels, gpn = (wg == kWgs - 1) ? kGPanelsMax : kGPanels;   // this warpgroup's panels of the 72-column accumulator
  {
    const float* gs = p.ds_last ? p.ds_last + static_cast<size_t>(bh) * hd * hd : nullptr;
    const float* gz = p.dz_last ? p.dz_last + static_cast<size_t>(bh) * hd : nullptr;
    float vals[kGPanelsMax * 8];   // all loads first: the TMEM stores below are compiler memory barriers
#pragma unroll
    for (int i = 0; i < kGPanelsMax * 8; ++i) {
      const int vcol = gp0 * 8 + i;
      float x = 0.f;
      if (upper && i < gpn * 8 && row < hd) {
        if (vcol < kD) x = (gs && vcol < hd) ? gs[vcol * hd + row] : 0.f;
        else if (vcol == kD) x = gz ? gz[row] : 0.f;
      }
      vals[i] = x;
    }
#pragma unroll
    for (int pn = 0; pn < kGPanelsMax; ++pn) {
      if (pn < gpn) {
        tmem_st8(lane_base + kColHi + (gp0 + pn) * 8, vals + pn * 8);
        if (upper) sm.g[(gp0 + pn) * kD + row] = pack8_bf16(vals + pn * 8);
      }
    }
    tmem_st_wait();
  }

  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint32_t id_kk = idesc_bf16(kC, kC, false, false);   // A, B contract over columns
  const uint32_t id_km = idesc_bf16(kC, kC, false, true);    // B contracts over rows
  const uint32_t id_mm = idesc_bf16(kC, kC, true, true);
  const uint32_t id_g = idesc_bf16(kD, kDX, true, true);
  bool timed_out = false;
  DoneFlags done_flags = load_done_flags(drow, (nchunks - 1) * kC, p.T, lane);
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

    // ---- the tiles have landed: feature map in place; keep-masked copies of phi(K) and V|1
    //      only if the chunk has a reset ----
    mbar_wait_flag(&sm.bar_load, it & 1, timed_out);
#pragma unroll
    for (int r = 0; r < 512 / kBwdThreads; ++r) {
      // element-wise, so the physical vector index serves (8 vectors = one token row)
      const int vid = r * kBwdThreads + tid;
      const int trow = vid >> 3;
      uint4 kv = sm.k[vid];
      if (p.feature_map && trow < valid) {
        // columns past the head dimension arrive as zeros and must stay zero (phi(0) = 1): the logical
        // 16-byte chunk of physical chunk `vid & 7` in row `trow` of a SW tile is (vid ^ trow) & 7
        const bool inside = kFull || ((vid ^ trow) & 7) < dpan;
        sm.q[vid] = inside ? phi8(sm.q[vid]) : zero4;
        kv = inside ? phi8(kv) : zero4;
        sm.k[vid] = kv;
      }
      if (has_reset) {
        const bool keep = row_keep(dm, trow);
        sm.kk[vid] = keep ? kv : zero4;
        sm.vk[vid] = keep ? sm.v[vid] : zero4;
      }
    }
    if (tid < kC) {
      const uint32_t one = tid < valid ? kOneBf16 : 0u;
      sm.vx[tid] = make_uint4(one, 0, 0, 0);
      if (has_reset) sm.vkx[tid] = make_uint4(row_keep(dm, tid) ? one : 0u, 0, 0, 0);
    }
    if (tid == 0) tma::wait_group_read<0>();   // the previous chunk's output tiles have left their staging buffers
    fence_smem_to_async();
    fence_before_sync();
    MXK_TB(1);
    __syncthreads();
    MXK_TB(7);

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
      if (leader) commit(&sm.bar[0]);
    }
    MXK_TB(8);
    mbar_wait_flag(&sm.bar[0], it & 1, timed_out);
    fence_after_sync();
    MXK_TB(2);

    // ---- epilogue 1: the four threads of a query row (two half-warps x two warpgroups) each
    //      cover 16 keys / state features; den and don are completed through shared memory ----
    {
      const bool live = row_live(dm, row);
      const int lo = row_first_key(dm, row);
      constexpr int KE = kKeysPerThread, PE = KE / 8;
      const int j0 = (upper ? 32 : 0) + wg * KE;   // first key / feature of this thread
      const int p0 = j0 >> 3;                      // and its first panel
      float s_dot = 0.f, z_dot = 0.f;
      {
        float rr[KE];
        tmem_ld_row<KE>(lane_base + kColR + wg * KE, rr);
#pragma unroll
        for (int pp = 0; pp < PE; ++pp) {
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
      float pv[KE], av[KE];
      tmem_ld_row<KE>(lane_base + kColP + wg * KE, pv);
      tmem_ld_row<KE>(lane_base + kColA + wg * KE, av);
      float den = live ? z_dot : 0.f, don = live ? s_dot : 0.f;
#pragma unroll
      for (int e = 0; e < KE; ++e) {
        const int j = j0 + e;
        const bool m = (j >= lo && j <= row);
        pv[e] = m ? pv[e] : 0.f;
        av[e] = m ? av[e] : 0.f;
        den += pv[e];
        don = fmaf(pv[e], av[e], don);
      }
      den += __shfl_xor_sync(0xffffffffu, den, 16);
      don += __shfl_xor_sync(0xffffffffu, don, 16);
      if (!upper) {
        sm.xch[wg][0][row] = den;
        sm.xch[wg][1][row] = don;
      }
      __syncthreads();
      // every thread of the row sums the warpgroups' partials in the same order: identical den / don in all of them
      den = sm.xch[0][0][row];
      don = sm.xch[0][1][row];
#pragma unroll
      for (int w = 1; w < kWgs; ++w) {
        den += sm.xch[w][0][row];
        don += sm.xch[w][1][row];
      }
      const float dcl = fmaxf(den, p.eps);
      const float inv = 1.f / dcl;
      const float dden = den > p.eps ? -don * inv * inv : 0.f;
#pragma unroll
      for (int jq = 0; jq < PE; ++jq) {
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
      // scaled dO rows: this thread's share of the eight panels, the extra column by one thread of the row
      const float sc = live ? inv : 0.f;
#pragma unroll
      for (int pp = 0; pp < PE; ++pp) {
        float f[8];
        unpack8_bf16(sm.d_o[sw_idx(row, p0 + pp)], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= sc;
        sm.dos[(p0 + pp) * kC + row] = pack8_bf16(f);
      }
      if (upper && wg == kWgs - 1) sm.dos[kPanels * kC + row] = make_uint4(pack_bf16(live ? dden : 0.f, 0.f), 0, 0, 0);
    }
    fence_smem_to_async();
    fence_before_sync();
    MXK_TB(3);
    __syncthreads();
    MXK_TB(9);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      // without a reset every key is kept: the unmasked tiles serve as the "keep" operands
      const Operand keep_k = sw_operand(smem_u32(has_reset ? sm.kk : sm.k), false);
      const Operand keep_v = sw_operand(smem_u32(has_reset ? sm.vk : sm.v), false);
      const Operand keep_vx{smem_u32(has_reset ? sm.vkx : sm.vx), kC, false};           // columns 64..79 of keep[V|1|0]
      const Operand g_k{smem_u32(sm.g), kD, false}, g_k4{smem_u32(sm.g) + 4 * 2 * kD * 16, kD, false};   // and G's K steps 0..3 / 4
      // dphiQ = dP phi(K) + dOs [S|z]                      (lower, columns 0..63)
      gemm<kC / 16>(tmem + kColLo, Operand{smem_u32(sm.dp), kC, false}, sw_operand(smem_u32(sm.k), true), id_km, false, leader);
      gemm<5>(tmem + kColLo, Operand{smem_u32(sm.dos), kC, false}, Operand{smem_u32(sm.s), kD, false}, id_kk, true, leader);
      // dphiK = dP^T phi(Q) + keep[V|1] [G|gz]^T           (upper, columns 0..63)
      gemm<kC / 16>(tmem + kUpper + kColLo, Operand{smem_u32(sm.dp), kC, true}, sw_operand(smem_u32(sm.q), true), id_mm, false, leader);
      gemm<4>(tmem + kUpper + kColLo, keep_v, g_k, id_kk, true, leader);
      gemm<1>(tmem + kUpper + kColLo, keep_vx, g_k4, id_kk, true, leader);
      // dV = (P/D)^T dO + keep phi(K) G^T                  (lower, columns 64..127)
      gemm<kC / 16>(tmem + kColHi, Operand{smem_u32(sm.pn), kC, true}, sw_operand(smem_u32(sm.d_o), true), id_mm, false, leader);
      gemm<kD / 16>(tmem + kColHi, keep_k, Operand{smem_u32(sm.g), kD, true}, id_km, true, leader);
      // [G|gz]^T = [no reset][G|gz]^T + phi(Q)^T dOs       (upper, columns 64..135)
      gemm<kC / 16>(tmem + kUpper + kColHi, sw_operand(smem_u32(sm.q), true), Operand{smem_u32(sm.dos), kC, true}, id_g, !has_reset, leader);
      if (leader) commit(&sm.bar[1]);
    }
    MXK_TB(10);
    // phi(Q) (lower) / phi(K) (upper) of this thread's columns, taken while the MMAs run
    constexpr int FE = kColsPerThread / 8;
    uint4 featv[FE];
    {
      const uint4* feat = upper ? sm.k : sm.q;
#pragma unroll
      for (int pn = 0; pn < FE; ++pn) featv[pn] = feat[sw_idx(row, wg * FE + pn)];
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.bar_free)) : "memory");
    }
    mbar_wait_flag(&sm.bar[1], it & 1, timed_out);
    fence_after_sync();
    if (tid == 0 && c > 0) {   // in flight while the output epilogue runs
      mbar_wait_flag(&sm.bar_free, it & 1, timed_out);
      issue_chunk_loads(c - 1);
    }
    MXK_TB(4);

    // ---- epilogue 2: every thread owns 32 (36, 40) columns of its row ----
    {
      // Output rows are staged as SW tiles in buffers the finished MMAs no longer need (dq in `dos`,
      // dk in `dp`, dv in `pn`) and leave by TMA stores after the chunk's last barrier; rows past the
      // end of the sequence are clipped by the tensor map.
      {
        // one stream: lower chains dphiQ through phi'(q) into dq, upper dphiK through phi'(k) into dk
        float acc[kColsPerThread];
        tmem_ld_row<kColsPerThread>(lane_base + kColLo + wg * kColsPerThread, acc);
        uint4 packed[FE];
#pragma unroll
        for (int pn = 0; pn < FE; ++pn) {
          float f[8];
          unpack8_bf16(featv[pn], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = acc[pn * 8 + e] * ((p.feature_map && f[e] <= 1.f) ? f[e] : 1.f);
          packed[pn] = pack8_bf16(f);
        }
        uint4* stage = upper ? sm.dp : sm.dos;
#pragma unroll
        for (int pn = 0; pn < FE; ++pn) stage[sw_idx(row, wg * FE + pn)] = packed[pn];
      }
      // one stream: lower stores dV, upper refreshes the bf16 operand copy of G | gz
      {
        float acc[kGPanelsMax * 8];
        if (wg < kWgs - 1) tmem_ld_row<kGPanels * 8>(lane_base + kColHi + gp0 * 8, acc);
        else tmem_ld_row<kGPanelsMax * 8>(lane_base + kColHi + gp0 * 8, acc);
        uint4 packed[kGPanelsMax];
#pragma unroll
        for (int pn = 0; pn < kGPanelsMax; ++pn)
          if (pn < gpn) packed[pn] = pack8_bf16(acc + pn * 8);
        if (upper) {
#pragma unroll
          for (int pn = 0; pn < kGPanelsMax; ++pn)
            if (pn < gpn) sm.g[(gp0 + pn) * kD + row] = packed[pn];
        }
        if (!upper) {   // dV: the first eight panels
#pragma unroll
          for (int pn = 0; pn < kGPanels; ++pn) sm.pn[sw_idx(row, gp0 + pn)] = packed[pn];
        }
        if (upper && c == 0 && row < hd) {
          float* out = p.ds0 ? p.ds0 + static_cast<size_t>(bh) * hd * hd : nullptr;
#pragma unroll
          for (int i = 0; i < kGPanelsMax * 8; ++i) {
            const int vcol = gp0 * 8 + i;
            if (i < gpn * 8) {
              if (vcol < kD) {
                if (out && vcol < hd) out[vcol * hd + row] = acc[i];
              } else if (vcol == kD && p.dz0) {
                p.dz0[static_cast<size_t>(bh) * hd + row] = acc[i];
              }
            }
          }
        }
      }
    }
    MXK_TB(5);
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_dq, sm.dos, t0, h, b);
      tma::store_plain_tile(&p.map_dk, sm.dp, t0, h, b);
      tma::store_plain_tile(&p.map_dv, sm.pn, t0, h, b);
      tma::commit_group();
    }
    MXK_TB(6);
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
extern "C" int mxk_debug_bwd_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_bwd_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_bwd_phase_cycles, 16 * sizeof(unsigned long long));
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
  if (d < 8 || d > kD || d % 8) return MXK_ERR_UNSUPPORTED;
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
  prm.d = d;
  // maps over the d-column tensors with 64-column boxes: the columns past d are zero-filled on loads and
  // clipped on stores
  if (!tma::make_sw_map(&prm.map_q, q, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_v, v, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_do, d_o, B, T, H, kC, d))
    return MXK_ERR_UNSUPPORTED;
  if (!tma::make_sw_map(&prm.map_dq, dq, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_dk, dk, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_dv, dv, B, T, H, kC, d))
    return MXK_ERR_UNSUPPORTED;
  auto kernel = d == kD ? linattn_bwd_kernel<true> : linattn_bwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(BwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  kernel<<<B * H, kBwdThreads, sizeof(BwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
