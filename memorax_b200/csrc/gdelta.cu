// Gated delta rule, forward, on the sm_100a tensor cores (math in gdelta_common.cuh).
//
// One CTA (256 threads, two warpgroups) owns one (batch, head) sequence and walks its
// 64-token chunks in order with the fp32 state S (128 x 128) resident in tensor memory;
// K, Q, V (128-byte-swizzled tiles) arrive by TMA one chunk ahead, as does the chunk's
// T' = (I + diag(beta) L)^-1 diag(beta) from the preparation kernel (gdelta_prep.cu), so the
// state-serial chain holds no triangular solve, only products:
//   MMAs 1: Q K^T (64 x 64, two key halves), Y^T = S_in K^T (128 x 64)
//   epilogue 1: tril(G o QK^T) (bf16), -(g Y)^T (bf16), Q and K rescaled in place (g Q, gam K)
//   MMAs 2: U^T = V^T T'^T - (g Y)^T T'^T  (128 x 64), i.e. U = T' (V - diag(g) K S_in^T)
//   epilogue 2: U^T as bf16 operand (and residual for the backward pass); S <- g_last S in place
//   MMAs 3: O^T = S_in (g Q)^T + U^T P^T (128 x 64), S += U^T (gam K) (128 x 128)
//   epilogue 3: output tile (one TMA store), bf16 operand copy of the new state.
#include <cstddef>

#include "gdelta_common.cuh"
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace gdelta;

struct FwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* alpha;
  const float* beta;
  const float* s0;
  const uint8_t* done;
  __nv_bfloat16* o;
  float* s_last;
  uint4* chunk_states;
  const uint4* tprime;        // T' of every chunk, written by the preparation kernel
  int* status;
  int B, T, H;
  int d;                      // head dimension in memory: 128, or 64 (the upper half of every tile is then the
                              // tensor maps' zero fill and the state's rows / columns 64..127 stay zero)
  CUtensorMap map_k, map_q, map_v;   // 64-token tiles as SW tiles (two 64-column blocks)
  CUtensorMap map_o;                 // 64-token tiles row-major
};

// What the kernel needs of a chunk's decay: no alpha / beta (beta is folded into T').
struct FwdDecay {
  float cum[kC], g[kC], gam[kC];
};

struct FwdSmem {
  uint4 s[kStateVecs];        // S_in bf16                      [k/8][v][8]
  uint4 k[kPanD * kC];        // K, after the first MMAs gam K  (SW tiles: two 64-column blocks)
  uint4 q[kPanD * kC];        // Q, after the first MMAs g Q    (SW tiles)
  uint4 v[kPanD * kC];        // V                              (SW tiles)
  uint4 yu[kPanC * kD];       // -(g Y)^T, then U^T [t/8][v][8], then the bf16 output tile [t][v] for the TMA store
  uint4 p[kPanC * kC];        // tril(G o QK^T)                 [j/8][t][8]
  uint4 tp[kAinvVecs];        // T'                             [j/8][t][8]
  FwdDecay cd;   // cd.gam doubles as the staging of log(alpha) while cum is being built
  uint64_t bar[3];
  uint64_t bar_load;
  uint32_t tmem;
};
static_assert(sizeof(FwdSmem) <= 113 * 1024, "two CTAs per SM");

// 256 TMEM columns per CTA (two CTAs per SM):
//   columns   0..127  S (fp32, all 128 lanes = value rows)
//   columns 128..191  Y^T = S_in K^T, afterwards U^T
//   columns 192..255  Q K^T (keys 0..31 in lanes 0..15 of each warp's quarter, keys 32..63 in lanes 16..31,
//                     32 columns), afterwards O^T (64 columns)
#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_gdf_phase_cycles[16];
namespace {
#define MXK_TF(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_gdf_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_TF(i) do {} while (0)
#endif
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kUpper = 16u << 16;
constexpr uint32_t kColS = 0, kColY = 128, kColU = 128, kColQK = 192, kColO = 192;

// 256 threads: two warpgroups that see the same TMEM lanes (warp w and warp w + 4 share a lane
// quarter) and split the columns of every row in the epilogues.
constexpr int kFwdThreads = 256;

__global__ void __launch_bounds__(kFwdThreads, 2) gdelta_fwd_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;            // warpgroup
  const int qw = warp & 3;             // TMEM lane quarter of this warp
  const int vt = tid & 127;            // value row owned in the transposed (M = 128) accumulators
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const bool upper = lane >= 16;
  const int row = qw * 16 + (lane & 15);  // token row owned in the M = 64 accumulators
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

  // carried state: thread (v, wg) owns S[v][64 wg .. 64 wg + 63]
  {
    const float* s0 = (p.s0 && vt < p.d && wg * 64 < p.d) ? p.s0 + (static_cast<size_t>(bh) * p.d + vt) * p.d + wg * 64 : nullptr;
    float vals[64];   // all loads first: the TMEM stores below are compiler memory barriers
#pragma unroll
    for (int c4 = 0; c4 < 16; ++c4) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s0) x = *reinterpret_cast<const float4*>(s0 + c4 * 4);
      vals[c4 * 4] = x.x; vals[c4 * 4 + 1] = x.y; vals[c4 * 4 + 2] = x.z; vals[c4 * 4 + 3] = x.w;
    }
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
      tmem_st8(lane_base + kColS + wg * 64 + c8 * 8, vals + c8 * 8);
      sm.s[(wg * 8 + c8) * kD + vt] = pack8_bf16(vals + c8 * 8);
    }
    tmem_st_wait();
  }

  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const size_t bt_base = static_cast<size_t>(b) * p.T;
  const uint32_t id_half = idesc_bf16(kC, 32, false, false);
  const uint32_t id_128x64 = idesc_bf16(kD, kC, false, false);
  const uint32_t id_vt = idesc_bf16(kD, kC, true, false);
  const uint32_t id_ds = idesc_bf16(kD, kD, false, true);
  constexpr uint32_t kBlk = kSwBlockVecs * 16;   // bytes between the two 64-column blocks of an SW tile pair
  bool timed_out = false;

  // K, Q, V (SW tiles) and T' of a chunk arrive by TMA / bulk copy, issued by one thread one chunk ahead: as
  // soon as the last MMA group of the previous chunk has released the buffers, so that the copies overlap
  // that chunk's output epilogue.
  auto issue_chunk_loads = [&](int cc) {
    fence_smem_to_async();   // earlier generic-proxy accesses to the buffers come first
    tma::expect_bytes(&sm.bar_load, (3 * kPanD * kC + kAinvVecs) * 16);
    tma::load_bulk(sm.tp, p.tprime + (static_cast<size_t>(bh) * nchunks + cc) * kAinvVecs, kAinvVecs * 16, &sm.bar_load);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, cc * kC, h, b, 0);
    tma::load_plain_tile(sm.k + kSwBlockVecs, &p.map_k, &sm.bar_load, cc * kC, h, b, 64);
    tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, cc * kC, h, b, 0);
    tma::load_plain_tile(sm.q + kSwBlockVecs, &p.map_q, &sm.bar_load, cc * kC, h, b, 64);
    tma::load_plain_tile(sm.v, &p.map_v, &sm.bar_load, cc * kC, h, b, 0);
    tma::load_plain_tile(sm.v + kSwBlockVecs, &p.map_v, &sm.bar_load, cc * kC, h, b, 64);
    if (cc + 1 < nchunks) {   // the chunk after it: into L2 now, so that its loads a chunk from now hit there
      tma::prefetch_plain_tile(&p.map_k, (cc + 1) * kC, h, b, 0);
      tma::prefetch_plain_tile(&p.map_q, (cc + 1) * kC, h, b, 0);
      tma::prefetch_plain_tile(&p.map_v, (cc + 1) * kC, h, b, 0);
      if (p.d > 64) {
        tma::prefetch_plain_tile(&p.map_k, (cc + 1) * kC, h, b, 64);
        tma::prefetch_plain_tile(&p.map_q, (cc + 1) * kC, h, b, 64);
        tma::prefetch_plain_tile(&p.map_v, (cc + 1) * kC, h, b, 64);
      }
      tma::prefetch_bulk(p.tprime + (static_cast<size_t>(bh) * nchunks + cc + 1) * kAinvVecs, kAinvVecs * 16);
    }
  };
  if (tid == 0) issue_chunk_loads(0);
  float alpha_next = 1.f;
  if (tid < kC && tid < p.T) alpha_next = __ldg(p.alpha + (bt_base + tid) * p.H + h);
  linattn::DoneFlags flags_next = linattn::load_done_flags(drow, 0, p.T, lane);

#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif
  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * kC;
    const uint64_t dm = linattn::done_mask_from_flags(flags_next);
    if (tid < kC) sm.cd.gam[tid] = __logf(alpha_next);
    fence_smem_to_async();   // the bf16 state copy written below / above is read by bulk copies and MMAs
    __syncthreads();
    // cum / g / gam of the chunk (same arithmetic as finish_chunk_decay)
    if (tid < 32) {
      const float l0 = sm.cd.gam[2 * tid], l1 = sm.cd.gam[2 * tid + 1];
      float s = l0 + l1;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, s, off);
        if (tid >= off) s += o;
      }
      sm.cd.cum[2 * tid] = s - l1;
      sm.cd.cum[2 * tid + 1] = s;
    }
    if (tid == 0 && p.chunk_states) {
      // residual for the backward pass: the state entering the chunk
      tma::store_bulk(p.chunk_states + (static_cast<size_t>(bh) * nchunks + c) * kResidualVecs, sm.s, kStateVecs * 16);
      tma::commit_group();
    }
    __syncthreads();
    if (tid < kC) {
      sm.cd.g[tid] = row_live(dm, tid) ? __expf(sm.cd.cum[tid]) : 0.f;
      sm.cd.gam[tid] = row_keep(dm, tid) ? __expf(sm.cd.cum[kC - 1] - sm.cd.cum[tid]) : 0.f;
    }
    MXK_TF(0);
    mbar_wait_flag(&sm.bar_load, c & 1, timed_out);
    // the previous chunk's output tile (the older bulk group) has left `yu` before epilogue 1 rewrites it
    if (tid == 0) { if (p.chunk_states) tma::wait_group_read<1>(); else tma::wait_group_read<0>(); }
    fence_before_sync();
    __syncthreads();
    MXK_TF(1);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand ak = sw_operand(smem_u32(sm.k), false, kBlk), aq = sw_operand(smem_u32(sm.q), false, kBlk);
      const Operand bk_hi = sw_operand(smem_u32(sm.k) + 32 * 128, false, kBlk);
      const Operand as{smem_u32(sm.s), kD, false};
      gemm128(tmem + kColQK, aq, ak, id_half, false, leader);               // Q K^T, keys 0..31  -> lanes 0..15
      gemm128(tmem + kUpper + kColQK, aq, bk_hi, id_half, false, leader);   // Q K^T, keys 32..63 -> lanes 16..31
      gemm128(tmem + kColY, as, ak, id_128x64, false, leader);              // Y^T = S_in K^T
      if (leader) commit(&sm.bar[0]);
    }
    mbar_wait_flag(&sm.bar[0], c & 1, timed_out);
    fence_after_sync();
    MXK_TF(2);

    // ---- epilogue 1: every thread turns 16 keys of its Q K^T row into the masked, decayed bf16 operand;
    //      thread (v, wg) turns 32 tokens of its Y^T row into -(g Y)^T; then Q and K are rescaled in place
    //      (g_t q_t for the inter-chunk output, gam_j k_j for the state update) ----
    {
      // every load first (TMEM, then the tile vectors and the decay scalars), so that their latencies overlap:
      // the TMEM accesses are compiler barriers, and stores into a tile would order the later loads from it
      const int j0 = (upper ? 32 : 0) + wg * 16;
      float qk[16], y[32];
      tmem_ld8(lane_base + kColQK + wg * 16, qk);
      tmem_ld8(lane_base + kColQK + wg * 16 + 8, qk + 8);
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) tmem_ld8(lane_base + kColY + wg * 32 + c8 * 8, y + c8 * 8);
      uint4* tile = upper ? sm.k : sm.q;
      uint4 tv[kPanD / 2];
#pragma unroll
      for (int p8 = 0; p8 < kPanD / 2; ++p8) tv[p8] = tile[sw_slot(row, wg * (kPanD / 2) + p8)];
      const float sc = upper ? sm.cd.gam[row] : sm.cd.g[row];
      const int lo = row_first_key(dm, row);
      const float cum_t = sm.cd.cum[row];
      float cj[16], gt[32];
#pragma unroll
      for (int e = 0; e < 16; ++e) cj[e] = sm.cd.cum[j0 + e];
#pragma unroll
      for (int e = 0; e < 32; ++e) gt[e] = sm.cd.g[wg * 32 + e];
      tmem_ld_wait();
#pragma unroll
      for (int jq = 0; jq < 2; ++jq) {
        float pm[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = j0 + jq * 8 + e;
          const bool in = (j >= lo && j <= row);
          pm[e] = in ? __expf(cum_t - cj[jq * 8 + e]) * qk[jq * 8 + e] : 0.f;
        }
        sm.p[((j0 >> 3) + jq) * kC + row] = pack8_bf16(pm);
      }
#pragma unroll
      for (int tp8 = 0; tp8 < 4; ++tp8) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = -gt[tp8 * 8 + e] * y[tp8 * 8 + e];
        sm.yu[(wg * 4 + tp8) * kD + vt] = pack8_bf16(f);
      }
#pragma unroll
      for (int p8 = 0; p8 < kPanD / 2; ++p8) {
        float f[8];
        unpack8_bf16(tv[p8], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= sc;
        tile[sw_slot(row, wg * (kPanD / 2) + p8)] = pack8_bf16(f);
      }
    }
    MXK_TF(3);
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();
    MXK_TF(4);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand av = sw_operand(smem_u32(sm.v), true, kBlk);     // V^T: contraction over the token rows
      const Operand ay{smem_u32(sm.yu), kD, false};
      const Operand bt{smem_u32(sm.tp), kC, false};
      gemm<kC / 16>(tmem + kColU, av, bt, id_vt, false, leader);          // U^T  = V^T T'^T
      gemm<kC / 16>(tmem + kColU, ay, bt, id_128x64, true, leader);       // U^T -= (g Y)^T T'^T
      if (leader) commit(&sm.bar[2]);
    }
    // meanwhile: S <- g_last S in place (the last MMAs of the previous chunk are long complete, the next
    // ones are issued after the barrier below); thread (v, wg) covers state columns 64 wg .. 64 wg + 63
    {
      fence_after_sync();
      const float g_last = sm.cd.g[kC - 1];
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        float s[32];
        tmem_ld_row<32>(lane_base + kColS + wg * 64 + q2 * 32, s);
#pragma unroll
        for (int e = 0; e < 32; ++e) s[e] *= g_last;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) tmem_st8(lane_base + kColS + wg * 64 + q2 * 32 + c8 * 8, s + c8 * 8);
      }
      tmem_st_wait();
    }
    mbar_wait_flag(&sm.bar[2], c & 1, timed_out);
    fence_after_sync();
    MXK_TF(5);

    // ---- epilogue 2: U^T as bf16 operand over -(g Y)^T (dead now) and as the backward pass's residual ----
    {
      uint4* res = p.chunk_states ? p.chunk_states + (static_cast<size_t>(bh) * nchunks + c) * kResidualVecs + kStateVecs : nullptr;
      float u[32];
      tmem_ld_row<32>(lane_base + kColU + wg * 32, u);
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        const uint4 u8 = pack8_bf16(u + jp * 8);
        sm.yu[(wg * 4 + jp) * kD + vt] = u8;
        if (res) res[(wg * 4 + jp) * kD + vt] = u8;
      }
    }
    MXK_TF(6);
    if (tid == 0) tma::wait_group_read<0>();   // the residual copy has finished reading `s` (rewritten in epilogue 3)
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand as{smem_u32(sm.s), kD, false}, bgq = sw_operand(smem_u32(sm.q), false, kBlk);
      const Operand au{smem_u32(sm.yu), kD, false}, bp{smem_u32(sm.p), kC, false};
      const Operand bgk = sw_operand(smem_u32(sm.k), true, kBlk);
      gemm128(tmem + kColO, as, bgq, id_128x64, false, leader);         // O^T  = S_in (g Q)^T
      gemm<kC / 16>(tmem + kColO, au, bp, id_128x64, true, leader);     // O^T += U^T P^T
      gemm<kC / 16>(tmem + kColS, au, bgk, id_ds, true, leader);        // S    = g_last S_in + U^T (gam K)
      if (leader) commit(&sm.bar[1]);
    }
    mbar_wait_flag(&sm.bar[1], c & 1, timed_out);
    fence_after_sync();
    MXK_TF(7);
    if (c + 1 < nchunks) {
      if (tid == 0) issue_chunk_loads(c + 1);
      alpha_next = 1.f;
      if (tid < kC && t0 + kC + tid < p.T) alpha_next = __ldg(p.alpha + (bt_base + t0 + kC + tid) * p.H + h);
      flags_next = linattn::load_done_flags(drow, t0 + kC, p.T, lane);
    }

    // ---- epilogue 3: output tile (staged row-major over U^T, dead now, for one TMA store), bf16 copy of the new state;
    //      thread (v, wg) covers tokens 32 wg .. 32 wg + 31 and state columns 64 wg .. 64 wg + 63 ----
    {
      __nv_bfloat16* otile = reinterpret_cast<__nv_bfloat16*>(sm.yu);
      float o[32], st[64];
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) tmem_ld8(lane_base + kColO + wg * 32 + c8 * 8, o + c8 * 8);
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) tmem_ld8(lane_base + kColS + wg * 64 + c8 * 8, st + c8 * 8);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) otile[(wg * 32 + e) * kD + vt] = __float2bfloat16(o[e]);
      const bool last = (c == nchunks - 1);
      float* sl = (last && p.s_last && vt < p.d && wg * 64 < p.d) ? p.s_last + (static_cast<size_t>(bh) * p.d + vt) * p.d + wg * 64 : nullptr;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        sm.s[(wg * 8 + c8) * kD + vt] = pack8_bf16(st + c8 * 8);
        if (sl) {
          *reinterpret_cast<float4*>(sl + c8 * 8) = make_float4(st[c8 * 8], st[c8 * 8 + 1], st[c8 * 8 + 2], st[c8 * 8 + 3]);
          *reinterpret_cast<float4*>(sl + c8 * 8 + 4) = make_float4(st[c8 * 8 + 4], st[c8 * 8 + 5], st[c8 * 8 + 6], st[c8 * 8 + 7]);
        }
      }
    }
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_o, sm.yu, t0, h, b);   // rows past the end of the sequence are clipped
      tma::commit_group();
    }
    MXK_TF(8);
  }
  if (tid == 0) tma::wait_group_all();

  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace mxk

#ifdef MXK_TIMING
extern "C" int mxk_debug_gdf_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_gdf_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_gdf_phase_cycles, 16 * sizeof(unsigned long long));
}
#endif

extern "C" {

size_t mxk_gdelta_chunk_states_bytes(int B, int T, int H, int d) {
  if (B <= 0 || T <= 0 || H <= 0 || (d != mxk::gdelta::kD && d != 64)) return 0;
  const size_t nchunks = (static_cast<size_t>(T) + mxk::gdelta::kC - 1) / mxk::gdelta::kC;
  return static_cast<size_t>(B) * H * nchunks * mxk::gdelta::kResidualVecs * sizeof(uint4);
}

size_t mxk_gdelta_workspace_bytes(int B, int T, int H, int d) {
  if (B <= 0 || T <= 0 || H <= 0 || (d != mxk::gdelta::kD && d != 64)) return 0;
  const size_t nchunks = (static_cast<size_t>(T) + mxk::gdelta::kC - 1) / mxk::gdelta::kC;
  return static_cast<size_t>(B) * H * nchunks * mxk::gdelta::kAinvVecs * sizeof(uint4);
}

int mxk_gdelta_bf16_fwd(const void* q, const void* k, const void* v, const float* alpha, const float* beta,
                        const float* s0, const uint8_t* done, void* o, float* s_last, void* chunk_states,
                        void* workspace, size_t workspace_bytes, int* status, int B, int T, int H, int d,
                        mxk_stream_t stream) {
  using namespace mxk;
  using namespace mxk::gdelta;
  if (!q || !k || !v || !alpha || !beta || !o) return MXK_ERR_NULL;
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d != kD && d != 64) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, (const void*)o, (const void*)chunk_states, (const void*)s0, (const void*)s_last})
    if (ptr && !aligned16(ptr)) return MXK_ERR_ALIGN;
  if (!workspace || workspace_bytes < mxk_gdelta_workspace_bytes(B, T, H, d)) return MXK_ERR_WORKSPACE;
  if (!aligned16(workspace)) return MXK_ERR_ALIGN;
  FwdParams prm;
  prm.q = static_cast<const __nv_bfloat16*>(q);
  prm.k = static_cast<const __nv_bfloat16*>(k);
  prm.v = static_cast<const __nv_bfloat16*>(v);
  prm.alpha = alpha;
  prm.beta = beta;
  prm.s0 = s0;
  prm.done = done;
  prm.o = static_cast<__nv_bfloat16*>(o);
  prm.s_last = s_last;
  prm.chunk_states = static_cast<uint4*>(chunk_states);
  prm.tprime = static_cast<const uint4*>(workspace);
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H; prm.d = d;
  if (!tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_q, q, B, T, H, kC, d) ||
      !tma::make_sw_map(&prm.map_v, v, B, T, H, kC, d) || !tma::make_plain_map(&prm.map_o, o, B, T, H, d, kC, kD))
    return MXK_ERR_UNSUPPORTED;
  const int st = launch_prep(k, alpha, beta, done, workspace, status, B, T, H, d, static_cast<cudaStream_t>(stream));
  if (st != MXK_OK) return st;
  cudaError_t e = cudaFuncSetAttribute(gdelta_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(FwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  gdelta_fwd_kernel<<<B * H, kFwdThreads, sizeof(FwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
