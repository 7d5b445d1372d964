// Chunked causal linear attention (ELU+1 feature map, carried state S and
// normaliser z, episode resets) on the sm_100a tensor cores.
//
// One CTA owns one (batch, head) sequence and walks its 64-token chunks in
// order.  The fp32 state S^T (d_k x d_v, plus the normaliser z as one extra
// column) stays resident in tensor memory for the whole sequence; every
// contraction is a tcgen05.mma over bf16 operands in shared memory (Q, K and the
// masked P as 128-byte-swizzled "SW tiles", V|1 and S^T|z in the panel format, both
// described in umma.cuh); Q, K, V arrive by TMA one chunk ahead:
//   P      = phi(Q) phi(K)^T                      (64 x 64,  K = d_k)
//   O      = live(phi(Q)) S_in^T                  (64 x 72,  K = d_k)
//   S^T    = [no reset] S^T + phi(K)^T keep(V|1)  (64 x 72,  K = 64 tokens)
//   O     += mask(P) (V|1)                        (64 x 72,  K = 64 tokens)
// The extra "1" column of V makes column 64 of O the normaliser phi(q).z, so
// numerator and denominator come out of the same accumulator.
// Resets inside a chunk: row i attends to keys j in [last reset <= i, i]; rows
// before the first reset also see the incoming state ("live"); only keys after
// the last reset ("keep") reach the outgoing state.
#include <cuda_bf16.h>

#include <cstddef>

#include "mxk_common.cuh"
#include "linattn_common.cuh"
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace linattn;

struct FwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* s0;
  const float* z0;
  const uint8_t* done;
  __nv_bfloat16* o;
  float* s_last;
  float* z_last;
  uint4* chunk_states;  // optional residual: bf16 S^T|z panels entering every chunk
  int* status;
  int B, T, H;
  int d;                // head dimension: a multiple of 8, at most kD; the tiles are kD wide, the rest zero
  float eps;
  int feature_map;
  int state_bulk;       // s0 / z0 are 16-byte aligned: they are staged through shared memory by bulk copies
  CUtensorMap map_q, map_k, map_o;   // 64-token tiles as SW tiles
  CUtensorMap map_v;          // 64-token tiles in panel order
};

struct FwdSmem {
  uint4 q[kPanels * kC];        // phi(Q), SW tile (128-byte-swizzled rows, umma.cuh)
  uint4 k[kPanels * kC];        // phi(K), SW tile; after the first MMAs: masked P, SW tile
  uint4 alt[kPanelsX * kC];     // chunks with a reset: keep rows of V|1 (panels), then live rows of phi(Q) (SW tile)
  uint4 v[kPanelsX * kC];       // V | 1                       [v/8][j]
  uint4 s[2][kPanelsX * kD];    // bf16 S^T | z entering / leaving the chunk   [v/8][k]
  uint64_t bar[2];
  uint64_t bar_load;
  uint64_t bar_state;
  uint32_t tmem;
};
static_assert(sizeof(FwdSmem) <= 55 * 1024, "four CTAs per SM");
static_assert(sizeof(FwdSmem::s) >= (kD * kD + kD) * sizeof(float), "the carried state is staged in s");
static_assert(offsetof(FwdSmem, k) % 1024 == 0 && offsetof(FwdSmem, alt) % 1024 == 0 && offsetof(FwdSmem, s) % 1024 == 0 &&
                  (kPanelsX * kD * 16) % 1024 == 0,
              "SW tiles are 1024-byte aligned");

// 128 TMEM columns per CTA.  M = 64 accumulators occupy 16 of the 32 lanes of a
// warp's TMEM quarter, so two of them share columns: P and later O in lanes
// 0..15 ("lower" threads, one query row each), the state S^T|z in lanes 16..31
// ("upper" threads, one key-feature row each).
#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_phase_cycles[16];
namespace {
#define MXK_T(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_T(i) do {} while (0)
#endif
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kUpper = 16u << 16;
#ifndef MXK_LINATTN_AHEAD
#define MXK_LINATTN_AHEAD 1
#endif
// Chunks whose tiles are requested into L2 ahead of their load.  One is the measured optimum at four chunks per
// sequence: requesting a whole sequence at its start (4) puts the first tiles behind the prefetch traffic of all
// resident CTAs and measured 7 % slower.
constexpr int kAhead = MXK_LINATTN_AHEAD;

// kFull: head dimension = the tile width (compile-time bounds); otherwise a multiple of 8 below it.
template <bool kFull>
__global__ void __launch_bounds__(kThreads, 4) linattn_fwd_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const bool upper = lane >= 16;
  const int row = warp * 16 + (lane & 15);   // lower: query row i; upper: state row k
  const int nchunks = (p.T + kC - 1) / kC;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  const int hd = kFull ? kD : p.d;   // head dimension
  const int dpan = hd >> 3;
#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_state, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  bool timed_out = false;
  MXK_T(11);
  // The carried state (d x d + d floats, contiguous per (batch, head)) comes in by two bulk copies into the
  // not-yet-used state buffers: 72 strided global loads per thread cost 7.5 k cycles per sequence here.
  float* const stage = reinterpret_cast<float*>(sm.s);
  const bool staged = p.state_bulk && (p.s0 || p.z0);
  if (staged && tid == 0) {
    tma::expect_bytes(&sm.bar_state, (p.s0 ? hd * hd * 4 : 0) + (p.z0 ? hd * 4 : 0));
    if (p.s0) tma::load_bulk(stage, p.s0 + static_cast<size_t>(bh) * hd * hd, hd * hd * 4, &sm.bar_state);
    if (p.z0) tma::load_bulk(stage + kD * kD, p.z0 + static_cast<size_t>(bh) * hd, hd * 4, &sm.bar_state);
  }

  // The raw Q, K, V tiles of a chunk arrive by TMA straight in operand order, issued by one
  // thread one chunk ahead: as soon as the second MMA group of the previous chunk has released
  // the buffers, so that the copies overlap that chunk's output epilogue.
  auto prefetch_chunk = [&](int cc) {
    tma::prefetch_plain_tile(&p.map_q, cc * kC, h, b);
    tma::prefetch_plain_tile(&p.map_k, cc * kC, h, b);
    tma::prefetch_panel_tile(&p.map_v, cc * kC, h, b);
  };
  auto issue_chunk_loads = [&](int cc) {
    fence_smem_to_async();   // earlier generic-proxy accesses to the buffers come first
    tma::expect_bytes(&sm.bar_load, 3 * kPanels * kC * 16);
    tma::load_plain_tile(sm.q, &p.map_q, &sm.bar_load, cc * kC, h, b);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, cc * kC, h, b);
    tma::load_panel_tile(sm.v, &p.map_v, &sm.bar_load, cc * kC, h, b);
    // a chunk kAhead positions on: into L2 now, so that its loads hit there -- except at the start of a sequence,
    // where every resident CTA asks for its first tiles and carried state at once and the prefetch only queues
    // in front of them (measured: 4 % of the forward)
    if (cc > 0 && cc + kAhead < nchunks) prefetch_chunk(cc + kAhead);
  };
  if (tid == 0) {
    issue_chunk_loads(0);
    for (int a = 1; a < kAhead && a < nchunks; ++a) prefetch_chunk(a);
  }

  // Carried state -> TMEM (fp32, upper lanes) and its bf16 operand copy.  Upper
  // thread `row` owns S^T[row][.] = S[.][row]; S is (d_v, d_k) row-major in
  // memory, so a fixed v is a coalesced read across threads.
  {
    const float* s0 = p.s0 ? p.s0 + static_cast<size_t>(bh) * hd * hd : nullptr;
    const float* z0 = p.z0 ? p.z0 + static_cast<size_t>(bh) * hd : nullptr;
    float vals[kDX];   // all loads first: the TMEM stores below are compiler memory barriers
    if (staged) {
      mbar_wait_flag(&sm.bar_state, 0, timed_out);
#pragma unroll
      for (int vcol = 0; vcol < kDX; ++vcol) {
        float x = 0.f;
        if (upper && row < hd) {
          if (vcol < kD) x = (s0 && vcol < hd) ? stage[vcol * hd + row] : 0.f;
          else if (vcol == kD) x = z0 ? stage[kD * kD + row] : 0.f;
        }
        vals[vcol] = x;
      }
      __syncthreads();   // every thread has taken its values before the bf16 copy overwrites the staging area
    } else {
#pragma unroll
      for (int vcol = 0; vcol < kDX; ++vcol) {
        float x = 0.f;
        if (upper && row < hd) {
          if (vcol < kD) x = (s0 && vcol < hd) ? s0[vcol * hd + row] : 0.f;
          else if (vcol == kD) x = z0 ? z0[row] : 0.f;
        }
        vals[vcol] = x;
      }
    }
#pragma unroll
    for (int pn = 0; pn < kPanelsX; ++pn) {
      tmem_st8(lane_base + pn * 8, vals + pn * 8);
      if (upper) sm.s[0][pn * kD + row] = pack8_bf16(vals + pn * 8);
    }
    tmem_st_wait();
  }
  MXK_T(12);

  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint32_t idesc_p = idesc_bf16(kC, kC, false, false);
  const uint32_t idesc_o = idesc_bf16(kC, kDX, false, true);
  const uint32_t idesc_s = idesc_bf16(kD, kDX, true, true);
  int cur = 0;
  MXK_T(9);
  DoneFlags done_flags = load_done_flags(drow, 0, p.T, lane);

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * kC;
    const int valid = min(kC, p.T - t0);
    const uint64_t dm = done_mask_from_flags(done_flags);
    done_flags = load_done_flags(drow, t0 + kC, p.T, lane);   // the next chunk's flags, needed a chunk from now
    const bool has_reset = dm != 0ull;
    MXK_T(0);

    // ---- the tiles have landed: feature map in place, keep-masked copy of V only if the
    //      chunk has a reset ----
    mbar_wait_flag(&sm.bar_load, c & 1, timed_out);
    MXK_T(8);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      // Q, K: element-wise, so the physical vector index serves (8 vectors = one token row)
      const int vid = r * kThreads + tid;
      if (p.feature_map && (vid >> 3) < valid) {
        // columns past the head dimension arrive as zeros and must stay zero (phi(0) = 1): the logical
        // 16-byte chunk of physical chunk `vid & 7` in row `vid >> 3` of a SW tile is (vid ^ (vid >> 3)) & 7
        const bool inside = kFull || ((vid ^ (vid >> 3)) & 7) < dpan;
        sm.q[vid] = inside ? phi8(sm.q[vid]) : zero4;
        sm.k[vid] = inside ? phi8(sm.k[vid]) : zero4;
      }
      if (has_reset) {
        int trow, seg;
        tile_vec(vid, trow, seg);
        const int slot = seg * kC + trow;
        sm.alt[slot] = row_keep(dm, trow) ? sm.v[slot] : zero4;
      }
    }
    if (tid < kC) {
      const uint4 one = make_uint4(tid < valid ? kOneBf16 : 0u, 0, 0, 0);
      sm.v[kPanels * kC + tid] = one;
      if (has_reset) sm.alt[kPanels * kC + tid] = row_keep(dm, tid) ? one : zero4;
    }
    if (tid == 0) tma::wait_group_read<0>();   // the previous output tile has left s[cur ^ 1], rewritten in epilogue A
    fence_smem_to_async();
    fence_before_sync();
    MXK_T(1);
    __syncthreads();
    MXK_T(2);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand aq = sw_operand(smem_u32(sm.q), false), bk = sw_operand(smem_u32(sm.k), false);
      const Operand ak = sw_operand(smem_u32(sm.k), true);
      const Operand bvk{smem_u32(has_reset ? sm.alt : sm.v), kC, true};
      gemm<kD / 16>(tmem, aq, bk, idesc_p, false, leader);                           // P        -> lower lanes
      gemm<kC / 16>(tmem + kUpper, ak, bvk, idesc_s, !has_reset, leader);            // S^T | z  -> upper lanes
      if (leader) commit(&sm.bar[0]);
      // residual for the backward pass: the state entering this chunk
      if (p.chunk_states && tid == 0) {
        tma::store_bulk(p.chunk_states + (static_cast<size_t>(bh) * nchunks + c) * (kPanelsX * kD), sm.s[cur],
                        kPanelsX * kD * 16);
        tma::commit_group();
      }
    }
    mbar_wait_flag(&sm.bar[0], c & 1, timed_out);
    fence_after_sync();
    MXK_T(3);

    // ---- epilogue A, one instruction stream for both halves: lower rows mask P into
    //      the bf16 A operand (over phi(K), which is dead now), upper rows convert the
    //      new state into the next chunk's bf16 B operand ----
    {
      float vals[kDX];
      tmem_ld_row<kDX>(lane_base, vals);
      const int lo = upper ? 0 : row_first_key(dm, row);
      const int hi = upper ? kDX : row;
#pragma unroll
      for (int pn = 0; pn < kPanelsX; ++pn) {
        float m[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = pn * 8 + e;
          m[e] = (j >= lo && j <= hi) ? vals[j] : 0.f;
        }
        // one store instruction for both halves
        uint4* dst = upper ? &sm.s[cur ^ 1][pn * kD + row] : &sm.k[sw_idx(row, pn & 7)];
        if (pn < kPanels || upper) *dst = pack8_bf16(m);
      }
      if (upper && c == nchunks - 1 && row < hd) {
        if (p.s_last) {
          float* out = p.s_last + static_cast<size_t>(bh) * hd * hd;
#pragma unroll
          for (int vcol = 0; vcol < kD; ++vcol)
            if (vcol < hd) out[vcol * hd + row] = vals[vcol];
        }
        if (p.z_last) p.z_last[static_cast<size_t>(bh) * hd + row] = vals[kD];
      }
    }
    if (has_reset) {   // live rows of phi(Q) for the inter-chunk product (the keep copy is dead now)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int vid = r * kThreads + tid;
        sm.alt[vid] = row_live(dm, vid >> 3) ? sm.q[vid] : zero4;
      }
    }
    if (tid == 0) tma::wait_group_read<0>();   // the residual copy has left s[cur], which stages the output below
    fence_smem_to_async();
    fence_before_sync();
    MXK_T(4);
    __syncthreads();
    MXK_T(5);

    if (warp == 0) {
      const bool leader = elect_one();
      fence_after_sync();
      const Operand aql = sw_operand(smem_u32(has_reset ? sm.alt : sm.q), false), bs{smem_u32(sm.s[cur]), kD, true};
      const Operand ap = sw_operand(smem_u32(sm.k), false), bv{smem_u32(sm.v), kC, true};
      gemm<kD / 16>(tmem, aql, bs, idesc_o, false, leader);     // O  = live(phi(Q)) S_in^T
      gemm<kC / 16>(tmem, ap, bv, idesc_o, true, leader);       // O += mask(P) (V|1)
      if (leader) commit(&sm.bar[1]);
    }
    mbar_wait_flag(&sm.bar[1], c & 1, timed_out);
    fence_after_sync();
    if (tid == 0 && c + 1 < nchunks) issue_chunk_loads(c + 1);
    MXK_T(6);

    // ---- epilogue B: lower rows normalise and store ----
    {
      float orow[kDX];
      tmem_ld_row<kDX>(lane_base, orow);
      const float inv = 1.f / fmaxf(orow[kD], p.eps);
      uint4 packed[kPanels];
#pragma unroll
      for (int pn = 0; pn < kPanels; ++pn) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = orow[pn * 8 + e] * inv;
        packed[pn] = pack8_bf16(f);
      }
      // s[cur] (the state that entered the chunk) is dead once the second MMA group has completed and
      // is not rewritten before the next chunk's first epilogue: it stages the output rows as an SW
      // tile for one TMA store (rows past the end of the sequence are clipped by the tensor map)
      if (!upper) {
#pragma unroll
        for (int pn = 0; pn < kPanels; ++pn) sm.s[cur][sw_idx(row, pn)] = packed[pn];
      }
    }
    fence_smem_to_async();
    __syncthreads();
    if (tid == 0) {
      tma::store_plain_tile(&p.map_o, sm.s[cur], t0, h, b);
      tma::commit_group();
    }
    cur ^= 1;
    MXK_T(7);
  }

  if (tid == 0) tma::wait_group_all();
  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
  MXK_T(10);
}

}  // namespace
}  // namespace mxk

#ifdef MXK_TIMING
extern "C" int mxk_debug_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_phase_cycles, 16 * sizeof(unsigned long long));
}
#endif

extern "C" {

size_t mxk_linattn_chunk_states_bytes(int B, int T, int H, int d) {
  if (B <= 0 || T <= 0 || H <= 0 || d < 8 || d > mxk::linattn::kD || d % 8) return 0;
  const size_t nchunks = (static_cast<size_t>(T) + mxk::linattn::kC - 1) / mxk::linattn::kC;
  return static_cast<size_t>(B) * H * nchunks * (mxk::linattn::kPanelsX * mxk::linattn::kD) * sizeof(uint4);
}

int mxk_linattn_bf16_fwd(const void* q, const void* k, const void* v, const float* s0, const float* z0,
                         const uint8_t* done, void* o, float* s_last, float* z_last, void* chunk_states,
                         int* status, int B, int T, int H, int d, float eps, int feature_map,
                         mxk_stream_t stream) {
  using namespace mxk;
  if (!q || !k || !v || !o) return MXK_ERR_NULL;
  if (B <= 0 || T <= 0 || H <= 0 || static_cast<long long>(B) * H > 0x7fffffffLL) return MXK_ERR_DIMS;
  if (d < 8 || d > kD || d % 8) return MXK_ERR_UNSUPPORTED;
  for (const void* ptr : {q, k, v, (const void*)o, (const void*)chunk_states})
    if (ptr && !aligned16(ptr)) return MXK_ERR_ALIGN;
  for (const void* ptr : {(const void*)s0, (const void*)z0, (const void*)s_last, (const void*)z_last})
    if (ptr && (reinterpret_cast<uintptr_t>(ptr) & 3u)) return MXK_ERR_ALIGN;
  FwdParams prm;
  prm.q = static_cast<const __nv_bfloat16*>(q);
  prm.k = static_cast<const __nv_bfloat16*>(k);
  prm.v = static_cast<const __nv_bfloat16*>(v);
  prm.s0 = s0;
  prm.z0 = z0;
  prm.done = done;
  prm.o = static_cast<__nv_bfloat16*>(o);
  prm.s_last = s_last;
  prm.z_last = z_last;
  prm.chunk_states = static_cast<uint4*>(chunk_states);
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H;
  prm.d = d;
  prm.eps = eps;
  prm.feature_map = feature_map;
  prm.state_bulk = (!s0 || aligned16(s0)) && (!z0 || aligned16(z0));
  // maps over the d-column tensors with 64-column boxes: the columns past d are zero-filled on loads and
  // clipped on stores
  if (!tma::make_sw_map(&prm.map_q, q, B, T, H, kC, d) || !tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d) ||
      !tma::make_panel_map(&prm.map_v, v, B, T, H, d, kC, kPanels) || !tma::make_sw_map(&prm.map_o, o, B, T, H, kC, d))
    return MXK_ERR_UNSUPPORTED;
  auto kernel = d == kD ? linattn_fwd_kernel<true> : linattn_fwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(FwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  kernel<<<B * H, kThreads, sizeof(FwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
