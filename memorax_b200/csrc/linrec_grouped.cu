// Real diagonal linear recurrence whose decay is shared by groups of channels:
//   h_t[c] = done_t ? b_t[c] : a_t[c / group] * h_{t-1}[c] + b_t[c]
// with a of shape (B, T, G) and D = G * group channels.  This is the scan of MambaCell
// (mamba.py:109-122: one scalar decay per (b, t, head) over a state_dim x head_dim matrix state) without
// expanding the decay to full width: the forward pass reads 4 + 4/group bytes per element instead of 8,
// and the backward pass reduces the decay gradient over each group in the kernel instead of writing a
// full-width tensor for the caller to sum.
//
// Same walk as linrec.cu: a thread owns 16 bytes of channels of one batch row and steps through time
// with several steps of loads in flight.  A warp covers 128 consecutive channels, and `group` is a
// multiple of 128, so a warp lies inside one group: the backward kernel reduces h_{t-1} g_t over the warp
// with shuffles and writes one partial per warp and step; a second small kernel adds the group / 128
// partials of a group in a fixed order (no atomics: results are bit-reproducible).
#include "mxk_common.cuh"

namespace mxk {
namespace {

constexpr int kBlockG = 256;

// kUnrollG time steps of loads are in flight per thread.  4 steps at four blocks per SM when the grid fills the
// machine; 8 steps at two blocks per SM (twice the registers) when it does not, so that a small batch still keeps
// enough bytes in flight per SM to cover the HBM latency.
// kLastOnly: `h` is (B, D) and receives the state after the last step only.
template <int kUnrollG, int kMinBlocks, bool kLastOnly = false>
__global__ void __launch_bounds__(kBlockG, kMinBlocks)
linrec_grouped_fwd_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ h0,
                          const float* __restrict__ a0, const uint8_t* __restrict__ done, float* __restrict__ h,
                          float* __restrict__ a_last, int B, int T, int D, int G, int group) {
  const int per_row = D / 4;
  const long long gid = static_cast<long long>(blockIdx.x) * kBlockG + threadIdx.x;
  if (gid >= static_cast<long long>(B) * per_row) return;
  const int bi = static_cast<int>(gid / per_row);
  const int col = static_cast<int>(gid % per_row) * 4;
  const int g = col / group;
  const size_t seq = static_cast<size_t>(bi) * T * D + col;
  const float* arow = a + static_cast<size_t>(bi) * T * G + g;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  float4 cur = h0 ? *reinterpret_cast<const float4*>(h0 + static_cast<size_t>(bi) * D + col) : make_float4(0.f, 0.f, 0.f, 0.f);
  // the decay leaf of the next carry, one value per group: written by the group's first thread
  const bool owns_decay = a_last != nullptr && (col % group) == 0;
  float acc = (owns_decay && a0) ? a0[static_cast<size_t>(bi) * G + g] : 1.f;

  for (int t0 = 0; t0 < T; t0 += kUnrollG) {
    float4 bv[kUnrollG];
    float av[kUnrollG];
    // The first loop only issues loads (a thread issues in order and would wait at the first use of a loaded
    // value): the reset bytes stay raw until the second loop.
    unsigned flag[kUnrollG];
#pragma unroll
    for (int u = 0; u < kUnrollG; ++u) {
      const int t = t0 + u;
      flag[u] = 0;
      if (t < T) {
        bv[u] = ld_stream(reinterpret_cast<const float4*>(b + seq + static_cast<size_t>(t) * D));
        av[u] = __ldg(arow + static_cast<size_t>(t) * G);
        if (drow) flag[u] = drow[t];
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollG; ++u) {
      const int t = t0 + u;
      if (t < T) {
        const bool reset = flag[u] != 0;
        const float at = reset ? 0.f : av[u];
        cur = make_float4(fmaf(at, cur.x, bv[u].x), fmaf(at, cur.y, bv[u].y), fmaf(at, cur.z, bv[u].z), fmaf(at, cur.w, bv[u].w));
        acc = reset ? av[u] : av[u] * acc;
        if constexpr (!kLastOnly) st_stream(reinterpret_cast<float4*>(h + seq + static_cast<size_t>(t) * D), cur);
      }
    }
  }
  if constexpr (kLastOnly) *reinterpret_cast<float4*>(h + static_cast<size_t>(bi) * D + col) = cur;
  if (owns_decay) a_last[static_cast<size_t>(bi) * G + g] = acc;
}

// Walks time right to left carrying c = a_{t+1} m_{t+1} g_{t+1}; the decay gradient of step t is the sum of
// h_{t-1} g_t over the group, of which this warp contributes one partial.
template <int kUnrollG, int kMinBlocks>
__global__ void __launch_bounds__(kBlockG, kMinBlocks)
linrec_grouped_bwd_kernel(const float* __restrict__ a, const float* __restrict__ h, const float* __restrict__ h0,
                          const uint8_t* __restrict__ done, const float* __restrict__ gh,
                          const float* __restrict__ gh_last, float* __restrict__ gb, float* __restrict__ ga_part,
                          float* __restrict__ gh0, int B, int T, int D, int G, int group) {
  const int per_row = D / 4;
  const long long gid = static_cast<long long>(blockIdx.x) * kBlockG + threadIdx.x;
  if (gid >= static_cast<long long>(B) * per_row) return;   // D % 128 == 0: whole warps leave together
  const int bi = static_cast<int>(gid / per_row);
  const int col = static_cast<int>(gid % per_row) * 4;
  const int g = col / group;
  const int wpg = group / 128;                 // warps per group
  const int wi = (col % group) / 128;          // this warp's slot among them
  const int lane = threadIdx.x & 31;
  const size_t seq = static_cast<size_t>(bi) * T * D + col;
  const size_t crow = static_cast<size_t>(bi) * D + col;
  const float* arow = a + static_cast<size_t>(bi) * T * G + g;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  float4 carry = gh_last ? *reinterpret_cast<const float4*>(gh_last + crow) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t0 = T - 1; t0 >= 0; t0 -= kUnrollG) {
    float4 gv[kUnrollG], hp[kUnrollG];
    float av[kUnrollG];
    // The first loop only issues loads: h_{t-1} is fetched whether or not step t resets, because a branch on the
    // reset byte would hold every later load back until that byte has arrived.
    unsigned flag[kUnrollG];
#pragma unroll
    for (int u = 0; u < kUnrollG; ++u) {
      const int t = t0 - u;
      flag[u] = 0;
      if (t >= 0) {
        const size_t off = seq + static_cast<size_t>(t) * D;
        gv[u] = ld_stream(reinterpret_cast<const float4*>(gh + off));
        av[u] = __ldg(arow + static_cast<size_t>(t) * G);
        if (drow) flag[u] = drow[t];
        hp[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ga_part) {
          if (t > 0) hp[u] = ld_stream(reinterpret_cast<const float4*>(h + off - D));
          else if (h0) hp[u] = *reinterpret_cast<const float4*>(h0 + crow);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollG; ++u) {
      const int t = t0 - u;
      if (t >= 0) {
        const bool reset = flag[u] != 0;
        const float4 gt = make_float4(gv[u].x + carry.x, gv[u].y + carry.y, gv[u].z + carry.z, gv[u].w + carry.w);
        st_stream(reinterpret_cast<float4*>(gb + seq + static_cast<size_t>(t) * D), gt);
        const float at = reset ? 0.f : av[u];
        carry = make_float4(at * gt.x, at * gt.y, at * gt.z, at * gt.w);
        if (ga_part) {
          float part = reset ? 0.f : (hp[u].x * gt.x + hp[u].y * gt.y) + (hp[u].z * gt.z + hp[u].w * gt.w);
#pragma unroll
          for (int off = 16; off >= 1; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
          if (lane == 0) ga_part[((static_cast<size_t>(bi) * T + t) * G + g) * wpg + wi] = part;
        }
      }
    }
  }
  if (gh0) *reinterpret_cast<float4*>(gh0 + crow) = carry;
}

// ga[i] = sum of the wpg partials of (b, t, group) i, in index order.
__global__ void __launch_bounds__(kBlockG)
sum_group_partials_kernel(const float* __restrict__ part, float* __restrict__ ga, long long n, int wpg) {
  const long long i = static_cast<long long>(blockIdx.x) * kBlockG + threadIdx.x;
  if (i >= n) return;
  float s = part[i * wpg];
  for (int w = 1; w < wpg; ++w) s += part[i * wpg + w];
  ga[i] = s;
}

int check_grouped(int B, int T, int D, int G) {
  if (B <= 0 || T <= 0 || D <= 0 || G <= 0) return MXK_ERR_DIMS;
  if (D % G != 0) return MXK_ERR_DIMS;
  if ((D / G) % 128 != 0) return MXK_ERR_UNSUPPORTED;   // a warp (32 threads x 4 channels) must lie inside one group
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

extern "C" {

size_t mxk_linrec_grouped_bwd_workspace_bytes(int B, int T, int D, int G) {
  if (mxk::check_grouped(B, T, D, G) != MXK_OK) return 0;
  const size_t wpg = static_cast<size_t>(D / G) / 128;
  return wpg > 1 ? static_cast<size_t>(B) * T * G * wpg * sizeof(float) : 0;
}

int mxk_linrec_f32_grouped_fwd(const float* a, const float* b, const float* h0, const float* a0, const uint8_t* done,
                               float* h, float* a_last, int B, int T, int D, int G, mxk_stream_t stream) {
  using namespace mxk;
  if (!a || !b || !h) return MXK_ERR_NULL;
  if (int st = check_grouped(B, T, D, G)) return st;
  for (const void* p : {(const void*)b, (const void*)h0, (const void*)h})
    if (p && !aligned16(p)) return MXK_ERR_ALIGN;
  for (const void* p : {(const void*)a, (const void*)a0, (const void*)a_last})
    if (p && (reinterpret_cast<uintptr_t>(p) & 3u)) return MXK_ERR_ALIGN;
  const long long threads = static_cast<long long>(B) * (D / 4);
  const unsigned blocks = static_cast<unsigned>((threads + kBlockG - 1) / kBlockG);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (blocks <= 3u * kNumSMs)
    linrec_grouped_fwd_kernel<8, 2><<<blocks, kBlockG, 0, s>>>(a, b, h0, a0, done, h, a_last, B, T, D, G, D / G);
  else
    linrec_grouped_fwd_kernel<4, 4><<<blocks, kBlockG, 0, s>>>(a, b, h0, a0, done, h, a_last, B, T, D, G, D / G);
  return launch_status();
}

int mxk_linrec_f32_grouped_last(const float* a, const float* b, const float* h0, const uint8_t* done, float* h_last,
                                int B, int T, int D, int G, mxk_stream_t stream) {
  using namespace mxk;
  if (!a || !b || !h_last) return MXK_ERR_NULL;
  if (int st = check_grouped(B, T, D, G)) return st;
  for (const void* p : {(const void*)b, (const void*)h0, (const void*)h_last})
    if (p && !aligned16(p)) return MXK_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(a) & 3u) return MXK_ERR_ALIGN;
  const long long threads = static_cast<long long>(B) * (D / 4);
  const unsigned blocks = static_cast<unsigned>((threads + kBlockG - 1) / kBlockG);
  linrec_grouped_fwd_kernel<8, 2, true><<<blocks, kBlockG, 0, static_cast<cudaStream_t>(stream)>>>(
      a, b, h0, nullptr, done, h_last, nullptr, B, T, D, G, D / G);
  return launch_status();
}

int mxk_linrec_f32_grouped_bwd(const float* a, const float* h, const float* h0, const uint8_t* done, const float* gh,
                               const float* gh_last, float* gb, float* ga, float* gh0, void* workspace,
                               size_t workspace_bytes, int B, int T, int D, int G, mxk_stream_t stream) {
  using namespace mxk;
  if (!a || !h || !gh || !gb) return MXK_ERR_NULL;
  if (int st = check_grouped(B, T, D, G)) return st;
  for (const void* p : {(const void*)h, (const void*)h0, (const void*)gh, (const void*)gh_last, (const void*)gb, (const void*)gh0})
    if (p && !aligned16(p)) return MXK_ERR_ALIGN;
  for (const void* p : {(const void*)a, (const void*)ga, (const void*)workspace})
    if (p && (reinterpret_cast<uintptr_t>(p) & 3u)) return MXK_ERR_ALIGN;
  const int wpg = (D / G) / 128;
  float* part = ga;   // one warp per group: its partial is the result
  if (ga && wpg > 1) {
    if (!workspace || workspace_bytes < mxk_linrec_grouped_bwd_workspace_bytes(B, T, D, G)) return MXK_ERR_WORKSPACE;
    part = static_cast<float*>(workspace);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long threads = static_cast<long long>(B) * (D / 4);
  const unsigned blocks = static_cast<unsigned>((threads + kBlockG - 1) / kBlockG);
  if (blocks <= 3u * kNumSMs)
    linrec_grouped_bwd_kernel<8, 2><<<blocks, kBlockG, 0, s>>>(a, h, h0, done, gh, gh_last, gb, part, gh0, B, T, D, G, D / G);
  else
    linrec_grouped_bwd_kernel<4, 4><<<blocks, kBlockG, 0, s>>>(a, h, h0, done, gh, gh_last, gb, part, gh0, B, T, D, G, D / G);
  if (int st = launch_status()) return st;
  if (ga && wpg > 1) {
    const long long n = static_cast<long long>(B) * T * G;
    sum_group_partials_kernel<<<static_cast<unsigned>((n + kBlockG - 1) / kBlockG), kBlockG, 0, s>>>(part, ga, n, wpg);
    return launch_status();
  }
  return MXK_OK;
}

}  // extern "C"
