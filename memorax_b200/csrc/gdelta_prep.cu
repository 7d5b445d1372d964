// Gated delta rule, chunk-parallel preparation: everything of the chunked form that does not depend on
// the carried state, computed for all chunks at once so that the state-serial kernels need no
// triangular solve.
//
// One CTA (128 threads) per (batch, head, 64-token chunk).  With the chunk quantities of
// gdelta_common.cuh (L = strict_tril(G o K K^T), A = I + diag(beta) L):
//   K K^T  on the tensor core (two N = 32 halves, so that each thread owns 32 keys of one token row),
//   N = -beta L in fp32 in shared memory, transposed,
//   A^-1 = (I - N)^-1 in fp32 by block recursion, every step using all four warps and no step longer than a
//          16-row chain: the four 16 x 16 diagonal blocks by forward substitution (one column per thread),
//          then  X_pq = X_pp N_pq X_qq  for the two 16 x 16 blocks under the diagonal of each 32 x 32 half,
//          then the same formula for the lower-left 32 x 32 block (the inverse of a block lower-triangular
//          matrix [[A11, 0], [A21, A22]] has -A22^-1 A21 A11^-1 there, and A21 = -N21).  A column-per-thread
//          substitution over all 64 rows would leave three warps idle behind a 63-step dependent chain.
//   T' = A^-1 diag(beta) leaves as bf16 in tensor-core operand order, [j/8][t][8] with t the row and
//          j the column.
// The forward kernel then forms U = T' (V - diag(g) K S_in^T) and the backward kernel dR = T'^T dU as
// plain tensor-core products.
#include "gdelta_common.cuh"
#include "tma.cuh"

namespace mxk {
namespace {

using namespace umma;
using namespace gdelta;

struct PrepParams {
  const float* alpha;
  const float* beta;
  const uint8_t* done;
  uint4* ainv;   // out: T', kAinvVecs uint4 per (b, h, chunk)
  int* status;
  int B, T, H, nchunks;
  CUtensorMap map_k;   // 64-token tiles as SW tiles (two 64-column blocks)
};

constexpr int kXS = kC + 1;   // row stride of the fp32 inverse: odd, so that a column walk is conflict-free

struct PrepSmem {
  // K, SW tiles (two 64-column blocks); once K K^T is done the same 16 KiB hold, in turn, the intermediate
  // products M = N_pq X_qq (fp32, [row][32]) and the staged bf16 T', [j/8][t][8]
  uint4 k[kPanD * kC];
  float lt[kC * kC];        // lt[j][t] = N[t][j] = -beta_t L_tj
  float x[kC * kXS];        // A^-1, row-major with stride kXS
  ChunkDecay cd;
  uint64_t bar_load, bar_mma;
  uint32_t tmem;
};
static_assert(sizeof(PrepSmem) <= 56 * 1024, "four CTAs per SM");

#ifdef MXK_TIMING
}  // namespace
__device__ unsigned long long g_gdp_phase_cycles[16];
namespace {
#define MXK_TP(i) do { if (tid == 0 && (blockIdx.x % 37) == 0) { const long long now_ = clock64(); atomicAdd(&g_gdp_phase_cycles[i], (unsigned long long)(now_ - t_prev_)); t_prev_ = now_; } } while (0)
#else
#define MXK_TP(i) do {} while (0)
#endif
constexpr uint32_t kPrepTmemCols = 32;
constexpr uint32_t kUpper = 16u << 16;

__global__ void __launch_bounds__(kThreads, 4) gdelta_prep_kernel(const __grid_constant__ PrepParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int item = blockIdx.x;
  const int c = item % p.nchunks, bh = item / p.nchunks, b = bh / p.H, h = bh % p.H;
  const int t0 = c * kC;
  const bool upper = lane >= 16;
  const int row = warp * 16 + (lane & 15);   // token row owned in the M = 64 accumulator

#ifdef MXK_TIMING
  long long t_prev_ = clock64();
#endif
  if (tid == 0) {
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kPrepTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  bool timed_out = false;
  MXK_TP(0);

  if (tid == 0) {
    tma::expect_bytes(&sm.bar_load, kPanD * kC * 16);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, t0, h, b, 0);
    tma::load_plain_tile(sm.k + kSwBlockVecs, &p.map_k, &sm.bar_load, t0, h, b, 64);
  }
  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint64_t dm = linattn::done_mask_from_flags(linattn::load_done_flags(drow, t0, p.T, lane));
  const float2 ab = fetch_chunk_decay(p.alpha, p.beta, static_cast<size_t>(b) * p.T, p.H, h, t0, p.T, tid);
  chunk_decay_from_regs(sm.cd, ab, dm, tid);
  MXK_TP(1);

  mbar_wait_flag(&sm.bar_load, 0, timed_out);
  MXK_TP(2);
  if (warp == 0) {
    const bool leader = elect_one();
    constexpr uint32_t kBlk = kSwBlockVecs * 16;
    const Operand ak = sw_operand(smem_u32(sm.k), false, kBlk);
    const Operand bk_hi = sw_operand(smem_u32(sm.k) + 32 * 128, false, kBlk);
    const uint32_t id_half = idesc_bf16(kC, 32, false, false);
    // keys 0..31 land in lanes 0..15 of each warp's TMEM quarter, keys 32..63 in lanes 16..31 of the same columns
    gemm128(tmem, ak, ak, id_half, false, leader);
    gemm128(tmem + kUpper, ak, bk_hi, id_half, false, leader);
    if (leader) commit(&sm.bar_mma);
  }
  mbar_wait_flag(&sm.bar_mma, 0, timed_out);
  fence_after_sync();
  MXK_TP(3);

  // -beta L, transposed: every thread owns 32 keys of its token row
  {
    const int lo = row_first_key(dm, row);
    const float cum_t = sm.cd.cum[row], beta_t = sm.cd.beta[row];
    const int j0 = upper ? 32 : 0;
    float kk[32];
    tmem_ld_row<32>(lane_base, kk);
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const int j = j0 + e;
      const bool in = (j >= lo && j < row);
      sm.lt[j * kC + row] = in ? -beta_t * __expf(cum_t - sm.cd.cum[j]) * kk[e] : 0.f;
    }
  }
  __syncthreads();

  MXK_TP(4);
  // ---- A^-1 = (I - N)^-1 by block recursion (N[t][j] = lt[j * kC + t]) ----
  float* const xm = sm.x;
  float* const mm = reinterpret_cast<float*>(sm.k);   // M, [row][32] (K is dead: K K^T has completed)
  for (int i = tid; i < kC * kXS; i += kThreads) xm[i] = 0.f;
  __syncthreads();
  // (1) the four 16 x 16 diagonal blocks: thread (p, c) solves column c of block p
  if (tid < kC) {
    const int p0 = (tid >> 4) * 16, c = tid & 15;
    float xc[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) xc[t] = (t == c) ? 1.f : 0.f;
#pragma unroll
    for (int jj = 0; jj < 15; ++jj) {
      const float uj = xc[jj];
#pragma unroll
      for (int t = jj + 1; t < 16; ++t) xc[t] = fmaf(sm.lt[(p0 + jj) * kC + p0 + t], uj, xc[t]);
    }
#pragma unroll
    for (int t = 0; t < 16; ++t) xm[(p0 + t) * kXS + p0 + c] = xc[t];
  }
  __syncthreads();
  // (2) X_pq = X_pp (N_pq X_qq) for (p, q) = (1, 0) and (3, 2): 64 threads per pair, thread = (row r, 4 columns)
  {
    const int pair = tid >> 6, r = tid & 15, c0 = ((tid >> 4) & 3) * 4;
    const int q0 = pair * 32, p0 = q0 + 16;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      const float a = sm.lt[(q0 + kk) * kC + p0 + r];          // N[p0 + r][q0 + kk]
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] = fmaf(a, xm[(q0 + kk) * kXS + q0 + c0 + e], acc[e]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) mm[(pair * 16 + r) * 32 + c0 + e] = acc[e];
    __syncthreads();
    float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      const float a = xm[(p0 + r) * kXS + p0 + kk];           // X_pp[r][kk]
#pragma unroll
      for (int e = 0; e < 4; ++e) out[e] = fmaf(a, mm[(pair * 16 + kk) * 32 + c0 + e], out[e]);
    }
    __syncthreads();   // every read of mm and of the diagonal blocks is done before anything is overwritten
#pragma unroll
    for (int e = 0; e < 4; ++e) xm[(p0 + r) * kXS + q0 + c0 + e] = out[e];
  }
  __syncthreads();
  // (3) the lower-left 32 x 32 block: X_PQ = X_PP (N_PQ X_QQ), thread = (row r of 32, 8 columns)
  {
    const int r = tid & 31, c0 = (tid >> 5) * 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      const float a = sm.lt[kk * kC + 32 + r];                 // N[32 + r][kk]
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(a, xm[kk * kXS + c0 + e], acc[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) mm[r * 32 + c0 + e] = acc[e];
    __syncthreads();
    float out[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = 0.f;
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      const float a = xm[(32 + r) * kXS + 32 + kk];            // X_PP[r][kk]
#pragma unroll
      for (int e = 0; e < 8; ++e) out[e] = fmaf(a, mm[kk * 32 + c0 + e], out[e]);
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; ++e) xm[(32 + r) * kXS + c0 + e] = out[e];
  }
  __syncthreads();
  MXK_TP(5);
  // T' = A^-1 diag(beta) as bf16, [j/8][t][8]: thread (t, half) packs four groups of eight columns
  {
    uint4* out = sm.k;
    const int t = tid & 63, g0 = (tid >> 6) * 4;
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int jcol = (g0 + gq) * 8 + e;
        f[e] = xm[t * kXS + jcol] * sm.cd.beta[jcol];
      }
      out[(g0 + gq) * kC + t] = pack8_bf16(f);
    }
  }
  fence_smem_to_async();
  __syncthreads();
  MXK_TP(6);
  if (tid == 0) {
    tma::store_bulk(p.ainv + static_cast<size_t>(item) * kAinvVecs, sm.k, kAinvVecs * 16);
    tma::commit_group();
    tma::wait_group_all();
  }
  MXK_TP(7);
  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kPrepTmemCols);
}

}  // namespace

#ifdef MXK_TIMING
}  // namespace mxk
extern "C" int mxk_debug_gdp_phase_cycles(unsigned long long* out, int reset) {
  if (reset) {
    unsigned long long z[16] = {};
    return (int)cudaMemcpyToSymbol(mxk::g_gdp_phase_cycles, z, sizeof(z));
  }
  return (int)cudaMemcpyFromSymbol(out, mxk::g_gdp_phase_cycles, 16 * sizeof(unsigned long long));
}
namespace mxk {
#endif

namespace gdelta {

int launch_prep(const void* k, const float* alpha, const float* beta, const uint8_t* done, void* ainv, int* status,
                int B, int T, int H, int d, cudaStream_t stream) {
  PrepParams prm;
  prm.alpha = alpha;
  prm.beta = beta;
  prm.done = done;
  prm.ainv = static_cast<uint4*>(ainv);
  prm.status = status;
  prm.B = B; prm.T = T; prm.H = H;
  prm.nchunks = (T + kC - 1) / kC;
  if (!tma::make_sw_map(&prm.map_k, k, B, T, H, kC, d)) return MXK_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(gdelta_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(PrepSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long items = static_cast<long long>(B) * H * prm.nchunks;
  if (items > 0x7fffffffLL) return MXK_ERR_DIMS;
  gdelta_prep_kernel<<<static_cast<unsigned>(items), kThreads, sizeof(PrepSmem), stream>>>(prm);
  return launch_status();
}

}  // namespace gdelta
}  // namespace mxk
