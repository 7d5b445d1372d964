// Chunked causal linear attention (ELU+1 feature map, carried state S and
// normaliser z, episode resets) on the sm_100a tensor cores.
//
// One CTA owns one (batch, head) sequence and walks its 64-token chunks in
// order.  The fp32 state S^T (d_k x d_v, plus the normaliser z as one extra
// column) stays resident in tensor memory for the whole sequence; every
// contraction is a tcgen05.mma over bf16 operands staged in shared memory in
// the panel format described in umma.cuh:
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

#include "mxk_common.cuh"
#include "linattn_common.cuh"

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
  float eps;
  int feature_map;
};

struct FwdSmem {
  uint4 q[kPanels * kC];     // phi(Q)            [k/8][i]
  uint4 ql[kPanels * kC];    // live rows only
  uint4 k[kPanels * kC];     // phi(K)            [k/8][j]
  uint4 v[kPanelsX * kC];    // V | 1             [v/8][j]
  uint4 vk[kPanelsX * kC];   // keep rows only
  uint4 p[kPanels * kC];     // masked P          [j/8][i]
  uint4 s[kPanelsX * kD];    // bf16 S^T | z      [v/8][k]
  uint64_t bar[2];
  uint32_t tmem;
};

constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColP = 0, kColO = 64, kColS = 136;

__global__ void __launch_bounds__(kThreads) linattn_fwd_kernel(const FwdParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int row = warp * 16 + (lane & 15);
  const bool row_active = lane < 16;
  const int nchunks = (p.T + kC - 1) / kC;

  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init_fence();
  }
  if (warp == 0) tmem_alloc(&sm.tmem, kTmemCols);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = sm.tmem;
  const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);

  // Carried state -> TMEM (fp32) and its bf16 operand copy.  Thread `row` owns
  // S^T[row][.] = S[.][row]; global S is (d_v, d_k) row-major, so a fixed v is a
  // coalesced read across threads.
  {
    const float* s0 = p.s0 ? p.s0 + static_cast<size_t>(bh) * kD * kD : nullptr;
    const float* z0 = p.z0 ? p.z0 + static_cast<size_t>(bh) * kD : nullptr;
#pragma unroll
    for (int pn = 0; pn < kPanelsX; ++pn) {
      float vals[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int vcol = pn * 8 + e;
        float x = 0.f;
        if (row_active) {
          if (vcol < kD) x = s0 ? s0[vcol * kD + row] : 0.f;
          else if (vcol == kD) x = z0 ? z0[row] : 0.f;
        }
        vals[e] = x;
      }
      tmem_st8(lane_base + kColS + pn * 8, vals);
      if (row_active) sm.s[pn * kD + row] = pack8_bf16(vals);
    }
    tmem_st_wait();
  }
  __syncthreads();
  if (p.chunk_states) {
    uint4* dst = p.chunk_states + static_cast<size_t>(bh) * nchunks * (kPanelsX * kD);
    for (int i = tid; i < kPanelsX * kD; i += kThreads) dst[i] = sm.s[i];
  }

  const size_t stride_t = static_cast<size_t>(p.H) * kD;
  const size_t seq_base = (static_cast<size_t>(b) * p.T * p.H + h) * kD;
  const uint8_t* drow = p.done ? p.done + static_cast<size_t>(b) * p.T : nullptr;
  const uint32_t idesc_p = idesc_bf16(kC, kC, false, false);
  const uint32_t idesc_o = idesc_bf16(kC, kDX, false, true);
  const uint32_t idesc_s = idesc_bf16(kD, kDX, true, true);
  bool timed_out = false;

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * kC;
    const int valid = min(kC, p.T - t0);
    const uint64_t dm = chunk_done_mask(drow, t0, p.T, lane);
    const bool has_reset = dm != 0ull;

    // ---- stage phi(Q), phi(K), V|1 (and their masked copies) ----
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int trow, seg;
      tile_vec(r * kThreads + tid, trow, seg);
      const bool in = trow < valid;
      const size_t g = seq_base + static_cast<size_t>(t0 + trow) * stride_t + seg * 8;
      uint4 qv = make_uint4(0, 0, 0, 0), kv = qv, vv = qv;
      if (in) {
        qv = __ldg(reinterpret_cast<const uint4*>(p.q + g));
        kv = __ldg(reinterpret_cast<const uint4*>(p.k + g));
        vv = __ldg(reinterpret_cast<const uint4*>(p.v + g));
        if (p.feature_map) {
          float f[8];
          unpack8_bf16(qv, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = phi(f[e]);
          qv = pack8_bf16(f);
          unpack8_bf16(kv, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = phi(f[e]);
          kv = pack8_bf16(f);
        }
      }
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const int slot = seg * kC + trow;
      sm.q[slot] = qv;
      sm.ql[slot] = row_live(dm, trow) ? qv : zero;
      sm.k[slot] = kv;
      sm.v[slot] = vv;
      sm.vk[slot] = row_keep(dm, trow) ? vv : zero;
    }
    if (tid < kC) {
      const uint4 one = make_uint4(tid < valid ? kOneBf16 : 0u, 0, 0, 0);
      sm.v[kPanels * kC + tid] = one;
      sm.vk[kPanels * kC + tid] = row_keep(dm, tid) ? one : make_uint4(0, 0, 0, 0);
    }
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    if (tid == 0) {
      fence_after_sync();
      const Operand aq{smem_u32(sm.q), kC, false}, aql{smem_u32(sm.ql), kC, false};
      const Operand bk{smem_u32(sm.k), kC, false}, ak{smem_u32(sm.k), kC, true};
      const Operand bs{smem_u32(sm.s), kD, true}, bvk{smem_u32(sm.vk), kC, true};
      gemm(tmem + kColP, aq, bk, idesc_p, kD / 16, false);
      gemm(tmem + kColO, aql, bs, idesc_o, kD / 16, false);
      gemm(tmem + kColS, ak, bvk, idesc_s, kC / 16, !has_reset);
      commit(&sm.bar[0]);
    }
    if (!mbar_wait(&sm.bar[0], c & 1)) timed_out = true;
    fence_after_sync();

    // ---- epilogue A: mask P -> bf16 operand; new state -> bf16 operand ----
    {
      float prow[kC];
      tmem_ld_row<kC>(lane_base + kColP, prow);
      const int lo = row_first_key(dm, row);
#pragma unroll
      for (int jp = 0; jp < kPanels; ++jp) {
        float m[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int j = jp * 8 + e;
          m[e] = (j >= lo && j <= row) ? prow[j] : 0.f;
        }
        if (row_active) sm.p[jp * kC + row] = pack8_bf16(m);
      }
      float srow[kDX];
      tmem_ld_row<kDX>(lane_base + kColS, srow);
      if (row_active) {
#pragma unroll
        for (int pn = 0; pn < kPanelsX; ++pn) sm.s[pn * kD + row] = pack8_bf16(srow + pn * 8);
        if (c == nchunks - 1) {
          if (p.s_last) {
            float* dst = p.s_last + static_cast<size_t>(bh) * kD * kD;
#pragma unroll
            for (int vcol = 0; vcol < kD; ++vcol) dst[vcol * kD + row] = srow[vcol];
          }
          if (p.z_last) p.z_last[static_cast<size_t>(bh) * kD + row] = srow[kD];
        }
      }
    }
    fence_smem_to_async();
    fence_before_sync();
    __syncthreads();

    if (tid == 0) {
      fence_after_sync();
      const Operand ap{smem_u32(sm.p), kC, false}, bv{smem_u32(sm.v), kC, true};
      gemm(tmem + kColO, ap, bv, idesc_o, kC / 16, true);
      commit(&sm.bar[1]);
    }
    if (p.chunk_states && c + 1 < nchunks) {
      uint4* dst = p.chunk_states + (static_cast<size_t>(bh) * nchunks + c + 1) * (kPanelsX * kD);
      for (int i = tid; i < kPanelsX * kD; i += kThreads) dst[i] = sm.s[i];
    }
    if (!mbar_wait(&sm.bar[1], c & 1)) timed_out = true;
    fence_after_sync();

    // ---- epilogue B: normalise and store ----
    {
      float orow[kDX];
      tmem_ld_row<kDX>(lane_base + kColO, orow);
      if (row_active && row < valid) {
        const float inv = 1.f / fmaxf(orow[kD], p.eps);
        uint4* dst = reinterpret_cast<uint4*>(p.o + seq_base + static_cast<size_t>(t0 + row) * stride_t);
#pragma unroll
        for (int pn = 0; pn < kPanels; ++pn) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = orow[pn * 8 + e] * inv;
          dst[pn] = pack8_bf16(f);
        }
      }
    }
  }

  if (timed_out && p.status) atomicExch(p.status, 1);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace
}  // namespace mxk

extern "C" {

size_t mxk_linattn_chunk_states_bytes(int B, int T, int H, int d) {
  if (B <= 0 || T <= 0 || H <= 0 || d != mxk::linattn::kD) return 0;
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
  if (d != kD) return MXK_ERR_UNSUPPORTED;
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
  prm.eps = eps;
  prm.feature_map = feature_map;
  static_assert(sizeof(FwdSmem) < 100 * 1024, "two CTAs per SM");
  cudaError_t e = cudaFuncSetAttribute(linattn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(sizeof(FwdSmem)));
  if (e != cudaSuccess) return static_cast<int>(e);
  linattn_fwd_kernel<<<B * H, kThreads, sizeof(FwdSmem), static_cast<cudaStream_t>(stream)>>>(prm);
  return launch_status();
}

}  // extern "C"
