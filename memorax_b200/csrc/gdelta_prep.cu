// Gated delta rule, chunk-parallel preparation: everything of the chunked form that does not depend on
// the carried state, computed for all chunks at once so that the state-serial kernels need no
// triangular solve.
//
// One CTA (128 threads) per (batch, head, 64-token chunk).  With the chunk quantities of
// gdelta_common.cuh (L = strict_tril(G o K K^T), A = I + diag(beta) L):
//   K K^T  on the tensor core (two N = 32 halves, so that each thread owns 32 keys of one token row),
//   -beta L in fp32 in shared memory, transposed,
//   A^-1   by forward substitution on the identity, one column per thread in fp32 registers
//          (columns 32..63 start at row 32: the upper-left of a unit lower-triangular inverse is zero),
//   T' = A^-1 diag(beta) leaves as bf16 in tensor-core operand order, [j/8][t][8] with t the row and
//          j the column.
// Six CTAs per SM (34 KiB of shared memory, 80 registers) overlap one chunk's copy and substitution latency
// with the others'.
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

struct PrepSmem {
  uint4 k[kPanD * kC];      // K, SW tiles (two 64-column blocks); once K K^T is done, its first 8 KiB stage
                            // the bf16 T', [j/8][t][8]
  float lt[kC * kC];        // lt[j][t] = -beta_t L_tj
  ChunkDecay cd;
  uint64_t bar_load, bar_mma;
  uint32_t tmem;
};
static_assert(sizeof(PrepSmem) <= 36 * 1024, "six CTAs per SM");

constexpr uint32_t kPrepTmemCols = 32;
constexpr uint32_t kUpper = 16u << 16;

__global__ void __launch_bounds__(kThreads, 6) gdelta_prep_kernel(const __grid_constant__ PrepParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int item = blockIdx.x;
  const int c = item % p.nchunks, bh = item / p.nchunks, b = bh / p.H, h = bh % p.H;
  const int t0 = c * kC;
  const bool upper = lane >= 16;
  const int row = warp * 16 + (lane & 15);   // token row owned in the M = 64 accumulator

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

  if (tid == 0) {
    tma::expect_bytes(&sm.bar_load, kPanD * kC * 16);
    tma::load_plain_tile(sm.k, &p.map_k, &sm.bar_load, t0, h, b, 0);
    tma::load_plain_tile(sm.k + kSwBlockVecs, &p.map_k, &sm.bar_load, t0, h, b, 64);
  }
  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint64_t dm = linattn::done_mask_from_flags(linattn::load_done_flags(drow, t0, p.T, lane));
  const float2 ab = fetch_chunk_decay(p.alpha, p.beta, static_cast<size_t>(b) * p.T, p.H, h, t0, p.T, tid);
  chunk_decay_from_regs(sm.cd, ab, dm, tid);

  mbar_wait_flag(&sm.bar_load, 0, timed_out);
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

  // A^-1 column by column: thread c < 64 solves A x = e_c
  if (warp < 2) {
    __align__(8) float r[kC];
#pragma unroll
    for (int t = 0; t < kC; ++t) r[t] = (t == tid) ? 1.f : 0.f;
    if (warp == 0) forward_substitute_range<0, kC - 1, kC>(reinterpret_cast<float2*>(r), sm.lt);
    else forward_substitute_range<32, kC - 1, kC>(reinterpret_cast<float2*>(r), sm.lt);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(sm.k);
    const int base = (tid >> 3) * kC * 8 + (tid & 7);   // element (t, j = tid) at [j/8][t][j%8]
    const float beta_j = sm.cd.beta[tid];                // column j of A^-1 times beta_j
#pragma unroll
    for (int t = 0; t < kC; ++t) out[base + t * 8] = __float2bfloat16(r[t] * beta_j);
  }
  fence_smem_to_async();
  __syncthreads();
  if (tid == 0) {
    tma::store_bulk(p.ainv + static_cast<size_t>(item) * kAinvVecs, sm.k, kAinvVecs * 16);
    tma::commit_group();
    tma::wait_group_all();
  }
  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kPrepTmemCols);
}

}  // namespace

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
