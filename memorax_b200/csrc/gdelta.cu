// Gated delta rule, forward, on the sm_100a tensor cores (math in gdelta_common.cuh).
//
// One CTA (256 threads, two warpgroups) owns one (batch, head) sequence and walks its
// 64-token chunks in order with the fp32 state S (128 x 128) resident in tensor memory;
// K, Q (128-byte-swizzled tiles) and V arrive by TMA one chunk ahead.  Per chunk:
//   MMAs 1: K K^T, Q K^T (64 x 64), Y^T = S_in K^T (128 x 64)
//   epilogue 1: row threads build -beta L (fp32, shared) and tril(G o QK^T) (bf16) and
//               rescale Q, K in place (g Q, gam K); warpgroup 0, thread v, forms its
//               column of beta (V - g Y) and solves the unit lower-triangular system by
//               forward substitution in fp32 registers while warpgroup 1 decays S in place
//   MMAs 2: O^T = S_in (g Q)^T + U^T P^T (128 x 64), S += U^T (gam K) (128 x 128)
//   epilogue 2: output tile (one TMA store), bf16 operand copy of the new state.
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
  int* status;
  int B, T, H;
  CUtensorMap map_k, map_q;   // 64-token tiles as SW tiles (two 64-column blocks)
  CUtensorMap map_v, map_o;   // 64-token tiles row-major
};

struct FwdSmem {
  uint4 s[kStateVecs];        // S_in bf16                      [k/8][v][8]
  uint4 k[kPanD * kC];        // K, after the first MMAs gam K  (SW tiles: two 64-column blocks)
  uint4 q[kPanD * kC];        // Q, after the first MMAs g Q    (SW tiles)
  uint4 vu[kC * 16];          // V row-major [t][v], then U^T   [j/8][v][8]
  uint4 p[kPanC * kC];        // tril(G o QK^T)                 [j/8][t][8]
  float lt[kC * kC];          // lt[j][t] = -beta_t L_tj, then the bf16 output tile [t][v]
  uint4 lb[4 * 32];           // bf16 copy of the off-diagonal block, rows t = 32..63, columns j = 0..31: [j/8][t-32][8]
  ChunkDecay cd;
  uint64_t bar[3];
  uint64_t bar_load;
  uint32_t tmem;
};
static_assert(sizeof(FwdSmem) <= 112 * 1024, "two CTAs per SM");

// 256 TMEM columns per CTA (two CTAs per SM):
//   columns   0..127  S (fp32, all 128 lanes = value rows)
//   columns 128..191  first K K^T (lanes 0..15 of each warp) and Q K^T (lanes 16..31),
//                     both M = 64; afterwards O^T (all lanes)
//   columns 192..255  Y^T = S_in K^T
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
constexpr uint32_t kColS = 0, kColKQ = 128, kColO = 128, kColY = 192;

// 256 threads: two warpgroups that see the same TMEM lanes (warp w and warp w + 4 share a lane
// quarter).  They split the columns of every row in the epilogues; around the forward
// substitution warpgroup 0 solves while warpgroup 1 decays the state.
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
    const float* s0 = p.s0 ? p.s0 + (static_cast<size_t>(bh) * kD + vt) * kD + wg * 64 : nullptr;
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
  const uint32_t id_64 = idesc_bf16(kC, kC, false, false);
  const uint32_t id_128x64 = idesc_bf16(kD, kC, false, false);
  const uint32_t id_ds = idesc_bf16(kD, kD, false, true);
  bool timed_out = false;

  // K, Q (SW tiles) and V (row-major) of a chunk arrive by TMA, issued by one thread
  // one chunk ahead: as soon as the second MMA group of the previous chunk has released
  // the buffers, so that the copies overlap that chunk's output epilogue.
  auto issue_chunk_loads = [&](int cc) {
    fence_smem_to_async();   // earlier generic-proxy accesses to the buffers come first
    tma::expect_bytes(&sm.bar_load, 3 * kPanD * kC * 16);
    // K, Q as SW tiles: two 64-column blocks of 64 x 128 bytes each
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, cc * kC, h, b, 0);
    tma::load_plain_tile(sm.k + kSwBlockVecs, &p.map_k, &sm.bar_load, cc * kC, h, b, 64);
    tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, cc * kC, h, b, 0);
    tma::load_plain_tile(sm.q + kSwBlockVecs, &p.map_q, &sm.bar_load, cc * kC, h, b, 64);
    tma::load_plain_tile(sm.vu, &p.map_v, &sm.bar_load, cc * kC, h, b);
  };
  if (tid == 0) issue_chunk_loads(0);
  float2 ab_next = fetch_chunk_decay(p.alpha, p.beta, bt_base, p.H, h, 0, p.T, tid);
  linattn::DoneFlags flags_next = linattn::load_done_flags(drow, 0, p.T, lane);

#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif
  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * kC;
    const uint64_t dm = linattn::done_mask_from_flags(flags_next);
    fence_smem_to_async();   // the bf16 state copy written below / above is read by bulk copies and MMAs
    __syncthreads();
    chunk_decay_from_regs(sm.cd, ab_next, dm, tid);
    if (tid == 0) {
      if (p.chunk_states) {
        // residual for the backward pass: the state entering the chunk
        tma::store_bulk(p.chunk_states + (static_cast<size_t>(bh) * nchunks + c) * kResidualVecs, sm.s, kStateVecs * 16);
        tma::commit_group();
      }
      // the previous chunk's output tile (older group) has left `lt` before epilogue 1a rewrites it
      if (p.chunk_states) tma::wait_group_read<1>(); else tma::wait_group_read<0>();
    }
    MXK_TF(0);
    mbar_wait_flag(&sm.bar_load, c & 1, timed_out);
    fence_before_sync();
    __syncthreads();
    MXK_TF(1);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand ak = sw_operand(smem_u32(sm.k), false, kSwBlockVecs * 16), aq = sw_operand(smem_u32(sm.q), false, kSwBlockVecs * 16);
      const Operand as{smem_u32(sm.s), kD, false};
      gemm128(tmem + kColKQ, ak, ak, id_64, false, leader);              // K K^T -> lower lanes
      gemm128(tmem + kUpper + kColKQ, aq, ak, id_64, false, leader);     // Q K^T -> upper lanes
      gemm128(tmem + kColY, as, ak, id_128x64, false, leader);           // Y^T = S_in K^T
      if (leader) commit(&sm.bar[0]);
    }
    mbar_wait_flag(&sm.bar[0], c & 1, timed_out);
    fence_after_sync();
    MXK_TF(2);

    // ---- epilogue 1a: lower lanes turn their K K^T row into -beta L (fp32), upper lanes their
    //      Q K^T row into the masked, decayed bf16 operand, 32 keys per warpgroup; then Q and K are
    //      rescaled in place (g_t q_t for the inter-chunk output, gam_j k_j for the state update),
    //      eight 16-byte vectors per thread ----
    {
      const int lo = row_first_key(dm, row);
      const float cum_t = sm.cd.cum[row], beta_t = sm.cd.beta[row];
      {
        float x[32];
        tmem_ld_row<32>(lane_base + kColKQ + wg * 32, x);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int j = wg * 32 + e;
          const bool in = (j >= lo && j <= row);
          x[e] *= in ? __expf(cum_t - sm.cd.cum[j]) : 0.f;
        }
        if (upper) {
#pragma unroll
          for (int jq = 0; jq < 4; ++jq) sm.p[(wg * 4 + jq) * kC + row] = pack8_bf16(x + jq * 8);
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int j = wg * 32 + e;
            x[e] = (j < row) ? -beta_t * x[e] : 0.f;
            sm.lt[j * kC + row] = x[e];
          }
          if (wg == 0 && row >= 32) {   // rows 32..63 x columns 0..31: operand of the blocked solve's MMA
#pragma unroll
            for (int jq = 0; jq < 4; ++jq) sm.lb[jq * 32 + (row - 32)] = pack8_bf16(x + jq * 8);
          }
        }
      }
      uint4* tile = upper ? sm.k : sm.q;
      const float sc = upper ? sm.cd.gam[row] : sm.cd.g[row];
#pragma unroll
      for (int p8 = 0; p8 < kPanD / 2; ++p8) {
        const int pn = wg * (kPanD / 2) + p8;
        float f[8];
        unpack8_bf16(tile[sw_slot(row, pn)], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= sc;
        tile[sw_slot(row, pn)] = pack8_bf16(f);
      }
    }
    MXK_TF(3);
    // ---- epilogue 1b.  Warpgroup 0, thread v: right-hand side and forward substitution for its
    //      column of U.  Warpgroup 1 meanwhile: S <- g_last S in place. ----
    __align__(8) float r[kC];
    if (wg == 0) {
      tmem_ld_row<kC>(lane_base + kColY, r);
#pragma unroll
      for (int t = 0; t < kC; ++t) r[t] = sm.cd.beta[t] * (bf16_at(sm.vu, t, vt) - sm.cd.g[t] * r[t]);
    } else {
      const float g_last = sm.cd.g[kC - 1];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        float s[32];
        tmem_ld_row<32>(lane_base + kColS + q4 * 32, s);
#pragma unroll
        for (int e = 0; e < 32; ++e) s[e] *= g_last;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) tmem_st8(lane_base + kColS + q4 * 32 + c8 * 8, s + c8 * 8);
      }
      tmem_st_wait();
    }
    fence_before_sync();
    __syncthreads();   // -beta L complete; V consumed (U^T reuses its buffer)
    MXK_TF(4);
    if (wg == 0) {
      // Blocked solve: rows 0..31 in fp32 registers; their effect on rows 32..63 (the 32 x 32
      // off-diagonal block times U_lo, a quarter of the FMAs and half of the dependent chain) on the
      // tensor core from the bf16 operands U_lo^T and -beta L, fp32 accumulate; then rows 32..63.
      uint4* res = p.chunk_states ? p.chunk_states + (static_cast<size_t>(bh) * nchunks + c) * kResidualVecs + kStateVecs : nullptr;
      forward_substitute_range<0, 31, 32>(reinterpret_cast<float2*>(r), sm.lt);
#pragma unroll
      for (int jp = 0; jp < kPanC / 2; ++jp) {
        const uint4 u8 = pack8_bf16(r + jp * 8);
        sm.vu[jp * kD + vt] = u8;
        if (res) res[jp * kD + vt] = u8;   // the backward pass reuses U instead of solving again
      }
      fence_smem_to_async();
      fence_before_sync();
      asm volatile("bar.sync 1, 128;" ::: "memory");   // warpgroup 0 only
      if (warp == 0) {
        const bool leader = elect_one();
        fence_after_sync();
        gemm<2>(tmem + kColKQ, Operand{smem_u32(sm.vu), kD, false}, Operand{smem_u32(sm.lb), 32, false},
                idesc_bf16(kD, 32, false, false), false, leader);
        if (leader) commit(&sm.bar[2]);
      }
      mbar_wait_flag(&sm.bar[2], c & 1, timed_out);
      fence_after_sync();
      {
        float delta[32];
        tmem_ld_row<32>(lane_base + kColKQ, delta);
#pragma unroll
        for (int e = 0; e < 32; ++e) r[32 + e] += delta[e];
      }
      forward_substitute_range<32, kC - 1, kC>(reinterpret_cast<float2*>(r), sm.lt);
#pragma unroll
      for (int jp = kPanC / 2; jp < kPanC; ++jp) {
        const uint4 u8 = pack8_bf16(r + jp * 8);
        sm.vu[jp * kD + vt] = u8;
        if (res) res[jp * kD + vt] = u8;
      }
    }
    MXK_TF(5);
    MXK_TF(6);
    if (tid == 0) tma::wait_group_read<0>();   // the residual copy has finished reading `s` (rewritten in epilogue 2)
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand as{smem_u32(sm.s), kD, false}, bgq = sw_operand(smem_u32(sm.q), false, kSwBlockVecs * 16);
      const Operand au{smem_u32(sm.vu), kD, false}, bp{smem_u32(sm.p), kC, false};
      const Operand bgk = sw_operand(smem_u32(sm.k), true, kSwBlockVecs * 16);
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
      ab_next = fetch_chunk_decay(p.alpha, p.beta, bt_base, p.H, h, t0 + kC, p.T, tid);
      flags_next = linattn::load_done_flags(drow, t0 + kC, p.T, lane);
    }

    // ---- epilogue 2: output tile (staged row-major for one TMA store), bf16 copy of the new state;
    //      thread (v, wg) covers tokens 32 wg .. 32 wg + 31 and state columns 64 wg .. 64 wg + 63 ----
    {
      __nv_bfloat16* otile = reinterpret_cast<__nv_bfloat16*>(sm.lt);
      {
        float o[32];
        tmem_ld_row<32>(lane_base + kColO + wg * 32, o);
#pragma unroll
        for (int e = 0; e < 32; ++e) otile[(wg * 32 + e) * kD + vt] = __float2bfloat16(o[e]);
      }
      const bool last = (c == nchunks - 1);
      float* sl = (last && p.s_last) ? p.s_last + (static_cast<size_t>(bh) * kD + vt) * kD : nullptr;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        const int q4 = wg * 2 + q2;
        float s[32];
        tmem_ld_row<32>(lane_base + kColS + q4 * 32, s);
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          sm.s[(q4 * 4 + c8) * kD + vt] = pack8_bf16(s + c8 * 8);
          if (sl) {
            *reinterpret_cast<float4*>(sl + q4 * 32 + c8 * 8) = make_float4(s[c8 * 8], s[c8 * 8 + 1], s[c8 * 8 + 2], s[c8 * 8 + 3]);
            *reinterpret_cast<float4*>(sl + q4 * 32 + c8 * 8 + 4) = make_float4(s[c8 * 8 + 4], s[c8 * 8 + 5], s[c8 * 8 + 6], s[c8 * 8 + 7]);
          }
        }
      }
    }
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_o, sm.lt, t0, h, b);   // rows past the end of the sequence are clipped
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
  if (B <= 0 || T <= 0 || H <= 0 || d != mxk::gdelta::kD) return 0;
  const size_t nchunks = (static_cast<size_t>(T) + mxk::gdelta::kC - 1) / mxk::gdelta::kC;
  return static_cast<size_t>(B) * H * nchunks * mxk::gdelta::kResidualVecs * sizeof(uint4);
}

int mxk_gdelta_bf16_fwd(const void* q, const void* k, const void* v, const float* alpha, const float* beta,
                        const float* s0, const uint8_t* done, void* o, float* s_last, void* chunk_states,
                        int* status, int B, int T, int H, int d, mxk_stream_t stream) {
  using namespace mxk;
  using namespace mxk::gdelta;
  if (!q || !k || !v || !alpha || !beta || !o) return MXK_ERR_NULL;
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d != kD) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, (const void*)o, (const void*)chunk_states, (const void*)s0, (const void*)s_last})
    if (ptr && !aligned16(ptr)) return MXK_ERR_ALIGN;
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
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H;
  if (!tma::make_sw_map(&prm.map_k, k, B, T, H, kC, kD) || !tma::make_sw_map(&prm.map_q, q, B, T, H, kC, kD) ||
      !tma::make_plain_map(&prm.map_v, v, B, T, H, kD, kC) || !tma::make_plain_map(&prm.map_o, o, B, T, H, kD, kC))
    return MXK_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(gdelta_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(FwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  gdelta_fwd_kernel<<<B * H, kFwdThreads, sizeof(FwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
