// Diagonal linear recurrences over time with carried state and episode resets:
// real fp32, complex64 and MinGRU's log-space form, forward and backward.
//
// All of these are bandwidth-bound: one pass over the (B,T,D) operands.  A
// thread owns 16 bytes of channels of one batch row and walks time
// sequentially, so a warp touches 512 contiguous bytes per step and a 256-
// thread block streams whole rows; loads for several time steps are issued
// before the dependent arithmetic so that enough bytes are in flight to cover
// HBM latency.  When B*D is too small to fill 148 SMs that way, each thread
// owns a single element instead (more, narrower threads).
#include <mutex>

#include "mxk_common.cuh"

namespace mxk {
namespace {

constexpr int kBlock = 256;
// Time steps whose loads are in flight together and the occupancy the
// register allocation must allow, per direction (tuned on B200: the one-read
// forward stream likes deep unrolling, the two-read backward stream likes more
// resident warps).
#ifndef MXK_LINREC_UNROLL_F
#define MXK_LINREC_UNROLL_F 4
#endif
#ifndef MXK_LINREC_MINB_F
#define MXK_LINREC_MINB_F 4
#endif
#ifndef MXK_LINREC_UNROLL_B
#define MXK_LINREC_UNROLL_B 2
#endif
#ifndef MXK_LINREC_MINB_B
#define MXK_LINREC_MINB_B 4
#endif
constexpr int kUnroll = 4;  // log-space kernels

template <int W> struct VecOf;
template <> struct VecOf<4> { using type = float4; };
template <> struct VecOf<2> { using type = float2; };
template <> struct VecOf<1> { using type = float; };

template <int W>
struct Pack {
  float v[W];
};

template <int W>
__device__ __forceinline__ Pack<W> load_pack(const float* p) {
  using V = typename VecOf<W>::type;
  V raw = ld_stream(reinterpret_cast<const V*>(p));
  Pack<W> out;
  const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
  for (int i = 0; i < W; ++i) out.v[i] = f[i];
  return out;
}

template <int W>
__device__ __forceinline__ Pack<W> load_pack_cached(const float* p) {
  using V = typename VecOf<W>::type;
  V raw = *reinterpret_cast<const V*>(p);
  Pack<W> out;
  const float* f = reinterpret_cast<const float*>(&raw);
#pragma unroll
  for (int i = 0; i < W; ++i) out.v[i] = f[i];
  return out;
}

template <int W>
__device__ __forceinline__ void store_pack(float* p, const Pack<W>& x) {
  using V = typename VecOf<W>::type;
  V raw;
  float* f = reinterpret_cast<float*>(&raw);
#pragma unroll
  for (int i = 0; i < W; ++i) f[i] = x.v[i];
  st_stream(reinterpret_cast<V*>(p), raw);
}

template <int W>
__device__ __forceinline__ Pack<W> fill_pack(float re, float im, bool cplx) {
  Pack<W> out;
#pragma unroll
  for (int i = 0; i < W; ++i) out.v[i] = (cplx && (i & 1)) ? im : re;
  return out;
}

// out = x * y (+ z), elementwise over the pack; complex packs hold (re, im) pairs.
template <bool CPLX, int W>
__device__ __forceinline__ Pack<W> mul(const Pack<W>& x, const Pack<W>& y) {
  Pack<W> o;
  if constexpr (CPLX) {
#pragma unroll
    for (int i = 0; i < W; i += 2) {
      o.v[i] = x.v[i] * y.v[i] - x.v[i + 1] * y.v[i + 1];
      o.v[i + 1] = x.v[i] * y.v[i + 1] + x.v[i + 1] * y.v[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) o.v[i] = x.v[i] * y.v[i];
  }
  return o;
}

template <bool CPLX, int W>
__device__ __forceinline__ Pack<W> mul_add(const Pack<W>& x, const Pack<W>& y, const Pack<W>& z) {
  Pack<W> o;
  if constexpr (CPLX) {
#pragma unroll
    for (int i = 0; i < W; i += 2) {
      o.v[i] = fmaf(x.v[i], y.v[i], fmaf(-x.v[i + 1], y.v[i + 1], z.v[i]));
      o.v[i + 1] = fmaf(x.v[i], y.v[i + 1], fmaf(x.v[i + 1], y.v[i], z.v[i + 1]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) o.v[i] = fmaf(x.v[i], y.v[i], z.v[i]);
  }
  return o;
}

// Complex conjugate of every (re, im) pair when `on` (no-op for real packs).
template <bool CPLX, int W>
__device__ __forceinline__ Pack<W> conj_if(Pack<W> x, int on) {
  if constexpr (CPLX) {
    if (on) {
#pragma unroll
      for (int i = 1; i < W; i += 2) x.v[i] = -x.v[i];
    }
  }
  return x;
}

template <int W>
__device__ __forceinline__ Pack<W> add(const Pack<W>& x, const Pack<W>& y) {
  Pack<W> o;
#pragma unroll
  for (int i = 0; i < W; ++i) o.v[i] = x.v[i] + y.v[i];
  return o;
}

// ------------------------------------------------------------------ forward
// Row stride is `row` floats (D for real, 2D for complex); a thread's W floats
// start at column `col`.
// kLastOnly: `h` is (B, row) and receives the state after the last step only (no per-step stores).
template <bool CPLX, int W, int kUnrollF = MXK_LINREC_UNROLL_F, int kMinBlocks = MXK_LINREC_MINB_F, bool kLastOnly = false>
__global__ void __launch_bounds__(kBlock, kMinBlocks)
linrec_fwd_kernel(const float* __restrict__ a, int a_tinv, const float* __restrict__ b,
                  const float* __restrict__ h0, const float* __restrict__ a0,
                  const uint8_t* __restrict__ done, float* __restrict__ h,
                  float* __restrict__ a_last, int B, int T, int row) {
  const int per_row = row / W;
  const long long gid = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  if (gid >= static_cast<long long>(B) * per_row) return;
  const int bi = static_cast<int>(gid / per_row);
  const int col = static_cast<int>(gid % per_row) * W;
  const size_t seq = static_cast<size_t>(bi) * T * row + col;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  Pack<W> cur = h0 ? load_pack_cached<W>(h0 + static_cast<size_t>(bi) * row + col) : fill_pack<W>(0.f, 0.f, CPLX);
  const bool want_decay = a_last != nullptr;
  Pack<W> acc = (want_decay && a0) ? load_pack_cached<W>(a0 + static_cast<size_t>(bi) * row + col)
                                   : fill_pack<W>(1.f, 0.f, CPLX);
  Pack<W> a_fix = fill_pack<W>(0.f, 0.f, CPLX);
  if (a_tinv) a_fix = load_pack_cached<W>(a + col);

  for (int t0 = 0; t0 < T; t0 += kUnrollF) {
    // Nothing in the first loop touches a loaded value (a thread issues in order and would wait for it there):
    // the reset bytes stay raw until the second loop.
    Pack<W> av[kUnrollF], bv[kUnrollF];
    unsigned flag[kUnrollF];
#pragma unroll
    for (int u = 0; u < kUnrollF; ++u) {
      const int t = t0 + u;
      flag[u] = 0;
      if (t < T) {
        const size_t off = seq + static_cast<size_t>(t) * row;
        bv[u] = load_pack<W>(b + off);
        if (!a_tinv) av[u] = load_pack<W>(a + off);
        if (drow) flag[u] = drow[t];
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollF; ++u) {
      const int t = t0 + u;
      if (t < T) {
        const Pack<W>& at = a_tinv ? a_fix : av[u];
        const bool reset = flag[u] != 0;
        cur = reset ? bv[u] : mul_add<CPLX, W>(at, cur, bv[u]);
        if (want_decay) acc = reset ? at : mul<CPLX, W>(at, acc);
        if constexpr (!kLastOnly) store_pack<W>(h + seq + static_cast<size_t>(t) * row, cur);
      }
    }
  }
  if constexpr (kLastOnly) {
    float* dst = h + static_cast<size_t>(bi) * row + col;
#pragma unroll
    for (int i = 0; i < W; ++i) dst[i] = cur.v[i];
  }
  if (want_decay) {
    float* dst = a_last + static_cast<size_t>(bi) * row + col;
#pragma unroll
    for (int i = 0; i < W; ++i) dst[i] = acc.v[i];
  }
}

// ------------------------------------------------------- time-split (small B*D)
// When there are too few channels to fill the machine with one thread per
// channel walking all of T, the time axis is split as well: a block owns
// 32 x W floats of a row (a warp reads 128 W contiguous bytes per step; a complex
// channel is one (re, im) pair) x 16 contiguous time segments.  Every thread loads
// its segment (<= L steps) into registers, folds it into an affine map (P, Q) with
// h_out = P h_in + Q (a reset makes P = 0), the sixteen maps of a channel are
// chained through shared memory, and each thread replays its segment from the right
// incoming state.  One pass over memory, T/16 sequential steps per thread.  `row`
// is the row length in floats (D for real, 2 D for complex).
constexpr int kSegs = 16;

template <bool CPLX, int L, int W>
__global__ void __launch_bounds__(32 * kSegs)
linrec_fwd_tsplit_kernel(const float* __restrict__ a, int a_tinv, const float* __restrict__ b,
                         const float* __restrict__ h0, const float* __restrict__ a0,
                         const uint8_t* __restrict__ done, float* __restrict__ h, float* __restrict__ a_last,
                         int B, int T, int row) {
  __shared__ float sp[kSegs][32 * W], sq[kSegs][32 * W], sd[kSegs][32 * W];
  __shared__ int sr[kSegs][32];
  const int cx = threadIdx.x & 31, seg = threadIdx.x >> 5;
  const long long ch = (static_cast<long long>(blockIdx.x) * 32 + cx) * W;   // first float = b * row + d
  const bool active = ch < static_cast<long long>(B) * row;
  const int bi = active ? static_cast<int>(ch / row) : 0, d = active ? static_cast<int>(ch % row) : 0;
  const int len = (T + kSegs - 1) / kSegs;
  const int t_begin = seg * len, t_end = min(T, t_begin + len);
  const size_t base = static_cast<size_t>(bi) * T * row + d;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  Pack<W> av[L], bv[L];
  unsigned flag[L];   // raw reset bytes: the load loop waits for no loaded value
  Pack<W> a_fix = fill_pack<W>(0.f, 0.f, CPLX);
  if (a_tinv && active) a_fix = load_pack_cached<W>(a + d);
#pragma unroll
  for (int i = 0; i < L; ++i) {
    const int t = t_begin + i;
    const bool in = active && t < t_end;
    bv[i] = in ? load_pack<W>(b + base + static_cast<size_t>(t) * row) : fill_pack<W>(0.f, 0.f, CPLX);
    av[i] = in ? (a_tinv ? a_fix : load_pack<W>(a + base + static_cast<size_t>(t) * row)) : fill_pack<W>(1.f, 0.f, CPLX);
    flag[i] = 0;
    if (in && drow) flag[i] = drow[t];
  }
  bool rs[L];
#pragma unroll
  for (int i = 0; i < L; ++i) rs[i] = flag[i] != 0;
  // segment summary: state map (P, Q); decay leaf: product since the last reset, and whether there was one
  Pack<W> P = fill_pack<W>(1.f, 0.f, CPLX), Q = fill_pack<W>(0.f, 0.f, CPLX), dec = fill_pack<W>(1.f, 0.f, CPLX);
  int had_reset = 0;
#pragma unroll
  for (int i = 0; i < L; ++i) {
    if (rs[i]) { P = fill_pack<W>(0.f, 0.f, CPLX); Q = bv[i]; dec = av[i]; had_reset = 1; }
    else { P = mul<CPLX, W>(P, av[i]); Q = mul_add<CPLX, W>(av[i], Q, bv[i]); dec = mul<CPLX, W>(dec, av[i]); }
  }
#pragma unroll
  for (int e = 0; e < W; ++e) {
    sp[seg][cx * W + e] = P.v[e];
    sq[seg][cx * W + e] = Q.v[e];
    sd[seg][cx * W + e] = dec.v[e];
  }
  sr[seg][cx] = had_reset;
  __syncthreads();
  Pack<W> hin = (active && h0) ? load_pack_cached<W>(h0 + static_cast<size_t>(bi) * row + d) : fill_pack<W>(0.f, 0.f, CPLX);
  for (int s2 = 0; s2 < seg; ++s2) {
    Pack<W> p2, q2;
#pragma unroll
    for (int e = 0; e < W; ++e) { p2.v[e] = sp[s2][cx * W + e]; q2.v[e] = sq[s2][cx * W + e]; }
    hin = mul_add<CPLX, W>(p2, hin, q2);
  }
#pragma unroll
  for (int i = 0; i < L; ++i) {
    const int t = t_begin + i;
    hin = rs[i] ? bv[i] : mul_add<CPLX, W>(av[i], hin, bv[i]);
    if (active && t < t_end) store_pack<W>(h + base + static_cast<size_t>(t) * row, hin);
  }
  if (a_last && seg == kSegs - 1 && active) {
    Pack<W> acc = a0 ? load_pack_cached<W>(a0 + static_cast<size_t>(bi) * row + d) : fill_pack<W>(1.f, 0.f, CPLX);
    for (int s2 = 0; s2 < kSegs; ++s2) {
      Pack<W> d2;
#pragma unroll
      for (int e = 0; e < W; ++e) d2.v[e] = sd[s2][cx * W + e];
      acc = sr[s2][cx] ? d2 : mul<CPLX, W>(acc, d2);
    }
#pragma unroll
    for (int e = 0; e < W; ++e) a_last[static_cast<size_t>(bi) * row + d + e] = acc.v[e];
  }
}

// The backward counterpart.  The carried cotangent c entering step t from the right obeys
// g_t = gh_t + c, c' = reset_t ? 0 : a_t g_t, so a segment is again an affine map c_out = P c_in + Q
// (walked right to left); the maps are chained from the last segment down, then every thread
// replays its segment, writing gb = g and the decay gradient (per step, or summed over its steps
// and then over the sixteen segments in a fixed order for a time-invariant decay).
template <bool CPLX, int L, int W>
__global__ void __launch_bounds__(32 * kSegs)
linrec_bwd_tsplit_kernel(const float* __restrict__ a, int a_tinv, const float* __restrict__ h,
                         const float* __restrict__ h0, const uint8_t* __restrict__ done,
                         const float* __restrict__ gh, const float* __restrict__ gh_last,
                         float* __restrict__ gb, float* __restrict__ ga, float* __restrict__ ga_partial,
                         float* __restrict__ gh0, int B, int T, int row, int conj_ops) {
  __shared__ float sp[kSegs][32 * W], sq[kSegs][32 * W];
  const int cx = threadIdx.x & 31, seg = threadIdx.x >> 5;
  const long long ch = (static_cast<long long>(blockIdx.x) * 32 + cx) * W;
  const bool active = ch < static_cast<long long>(B) * row;
  const int bi = active ? static_cast<int>(ch / row) : 0, d = active ? static_cast<int>(ch % row) : 0;
  const int len = (T + kSegs - 1) / kSegs;
  const int t_begin = seg * len, t_end = min(T, t_begin + len);
  const size_t base = static_cast<size_t>(bi) * T * row + d;
  const size_t crow = static_cast<size_t>(bi) * row + d;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;
  const bool want_ga = (ga != nullptr) || (ga_partial != nullptr);

  // The load loop issues every load of the segment, h_{t-1} for the decay gradient included, and waits for none
  // (a thread issues in order): conjugation and the reset test follow in a loop of their own.
  Pack<W> av[L], gv[L], hp[L];
  unsigned flag[L];
  Pack<W> a_fix = fill_pack<W>(0.f, 0.f, CPLX);
  if (a_tinv && active) a_fix = load_pack_cached<W>(a + d);
#pragma unroll
  for (int i = 0; i < L; ++i) {
    const int t = t_begin + i;
    const bool in = active && t < t_end;
    const size_t off = base + static_cast<size_t>(t) * row;
    gv[i] = in ? load_pack<W>(gh + off) : fill_pack<W>(0.f, 0.f, CPLX);
    av[i] = in ? (a_tinv ? a_fix : load_pack<W>(a + off)) : fill_pack<W>(1.f, 0.f, CPLX);
    flag[i] = 0;
    if (in && drow) flag[i] = drow[t];
    hp[i] = fill_pack<W>(0.f, 0.f, CPLX);
    if (in && want_ga) {
      if (t > 0) hp[i] = load_pack<W>(h + off - row);
      else if (h0) hp[i] = load_pack_cached<W>(h0 + crow);
    }
  }
  bool rs[L];
#pragma unroll
  for (int i = 0; i < L; ++i) {
    rs[i] = flag[i] != 0;
    av[i] = conj_if<CPLX, W>(av[i], conj_ops);
  }
  Pack<W> P = fill_pack<W>(1.f, 0.f, CPLX), Q = fill_pack<W>(0.f, 0.f, CPLX);
#pragma unroll
  for (int i = L - 1; i >= 0; --i) {
    if (rs[i]) { P = fill_pack<W>(0.f, 0.f, CPLX); Q = P; }
    else { P = mul<CPLX, W>(av[i], P); Q = mul<CPLX, W>(av[i], add<W>(gv[i], Q)); }
  }
#pragma unroll
  for (int e = 0; e < W; ++e) {
    sp[seg][cx * W + e] = P.v[e];
    sq[seg][cx * W + e] = Q.v[e];
  }
  __syncthreads();
  Pack<W> carry = (active && gh_last) ? load_pack_cached<W>(gh_last + crow) : fill_pack<W>(0.f, 0.f, CPLX);
  for (int s2 = kSegs - 1; s2 > seg; --s2) {
    Pack<W> p2, q2;
#pragma unroll
    for (int e = 0; e < W; ++e) { p2.v[e] = sp[s2][cx * W + e]; q2.v[e] = sq[s2][cx * W + e]; }
    carry = mul_add<CPLX, W>(p2, carry, q2);
  }
  __syncthreads();   // sp is reused for the decay-gradient partials
  Pack<W> ga_acc = fill_pack<W>(0.f, 0.f, CPLX);
#pragma unroll
  for (int i = L - 1; i >= 0; --i) {
    const int t = t_begin + i;
    const bool in = active && t < t_end;
    const size_t off = base + static_cast<size_t>(t) * row;
    const Pack<W> g = add<W>(gv[i], carry);
    if (in) store_pack<W>(gb + off, g);
    if (rs[i]) {
      carry = fill_pack<W>(0.f, 0.f, CPLX);
      if (want_ga && !a_tinv) store_pack<W>(ga + off, carry);
    } else if (in) {
      carry = mul<CPLX, W>(av[i], g);
      if (want_ga) {
        const Pack<W> hc = conj_if<CPLX, W>(hp[i], conj_ops);
        if (a_tinv) ga_acc = mul_add<CPLX, W>(hc, g, ga_acc);
        else store_pack<W>(ga + off, mul<CPLX, W>(hc, g));
      }
    }
  }
  if (gh0 && seg == 0 && active) {
#pragma unroll
    for (int e = 0; e < W; ++e) gh0[crow + e] = carry.v[e];
  }
  if (a_tinv && ga_partial) {
#pragma unroll
    for (int e = 0; e < W; ++e) sp[seg][cx * W + e] = ga_acc.v[e];
    __syncthreads();
    if (seg == 0 && active) {
#pragma unroll
      for (int e = 0; e < W; ++e) {
        float t = sp[kSegs - 1][cx * W + e];
        for (int s2 = kSegs - 2; s2 >= 0; --s2) t += sp[s2][cx * W + e];
        ga_partial[crow + e] = t;
      }
    }
  }
}

// ----------------------------------------------------------------- backward
// Walks time right to left carrying c = a_{t+1} m_{t+1} g_{t+1}.
template <bool CPLX, int W, int kUnrollB = MXK_LINREC_UNROLL_B, int kMinBlocks = MXK_LINREC_MINB_B>
__global__ void __launch_bounds__(kBlock, kMinBlocks)
linrec_bwd_kernel(const float* __restrict__ a, int a_tinv, const float* __restrict__ h,
                  const float* __restrict__ h0, const uint8_t* __restrict__ done,
                  const float* __restrict__ gh, const float* __restrict__ gh_last,
                  float* __restrict__ gb, float* __restrict__ ga, float* __restrict__ ga_partial,
                  float* __restrict__ gh0, int B, int T, int row, int conj_ops) {
  const int per_row = row / W;
  const long long gid = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  if (gid >= static_cast<long long>(B) * per_row) return;
  const int bi = static_cast<int>(gid / per_row);
  const int col = static_cast<int>(gid % per_row) * W;
  const size_t seq = static_cast<size_t>(bi) * T * row + col;
  const size_t crow = static_cast<size_t>(bi) * row + col;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  Pack<W> carry = gh_last ? load_pack_cached<W>(gh_last + crow) : fill_pack<W>(0.f, 0.f, CPLX);
  Pack<W> a_fix = fill_pack<W>(0.f, 0.f, CPLX);
  if (a_tinv) a_fix = conj_if<CPLX, W>(load_pack_cached<W>(a + col), conj_ops);
  Pack<W> ga_acc = fill_pack<W>(0.f, 0.f, CPLX);
  const bool want_ga = (ga != nullptr) || (ga_partial != nullptr);

  for (int t0 = T - 1; t0 >= 0; t0 -= kUnrollB) {
    // The first loop only issues loads: a thread issues in order, so a conjugation, a comparison or a branch on
    // a loaded value there would hold every later load back by one trip to memory per step.  h_{t-1} is therefore
    // fetched whether or not step t resets, and conjugation and the reset test wait for the second loop.
    Pack<W> av[kUnrollB], gv[kUnrollB], hp[kUnrollB];
    unsigned flag[kUnrollB];
#pragma unroll
    for (int u = 0; u < kUnrollB; ++u) {
      const int t = t0 - u;
      flag[u] = 0;
      if (t >= 0) {
        const size_t off = seq + static_cast<size_t>(t) * row;
        gv[u] = load_pack<W>(gh + off);
        if (!a_tinv) av[u] = load_pack<W>(a + off);
        if (drow) flag[u] = drow[t];
        if (want_ga) {
          if (t > 0) hp[u] = load_pack<W>(h + off - row);
          else hp[u] = h0 ? load_pack_cached<W>(h0 + crow) : fill_pack<W>(0.f, 0.f, CPLX);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnrollB; ++u) {
      const int t = t0 - u;
      if (t >= 0) {
        const Pack<W> g = add<W>(gv[u], carry);
        const size_t off = seq + static_cast<size_t>(t) * row;
        store_pack<W>(gb + off, g);
        if (flag[u] != 0) {
          carry = fill_pack<W>(0.f, 0.f, CPLX);
          if (want_ga && !a_tinv) store_pack<W>(ga + off, carry);
        } else {
          const Pack<W> at = a_tinv ? a_fix : conj_if<CPLX, W>(av[u], conj_ops);
          carry = mul<CPLX, W>(at, g);
          if (want_ga) {
            const Pack<W> hc = conj_if<CPLX, W>(hp[u], conj_ops);
            if (a_tinv) ga_acc = mul_add<CPLX, W>(hc, g, ga_acc);
            else store_pack<W>(ga + off, mul<CPLX, W>(hc, g));
          }
        }
      }
    }
  }
  if (gh0) {
#pragma unroll
    for (int i = 0; i < W; ++i) gh0[crow + i] = carry.v[i];
  }
  if (a_tinv && ga_partial) {
#pragma unroll
    for (int i = 0; i < W; ++i) ga_partial[crow + i] = ga_acc.v[i];
  }
}

// Sums the (B, row) per-sequence partials of the time-invariant decay gradient
// over the batch in a fixed order (deterministic; no atomics).  A block owns 32
// columns; its eight thread rows each sum every eighth sequence, then thread row
// 0 adds the eight partials in order.
__global__ void __launch_bounds__(kBlock)
reduce_rows_kernel(const float* __restrict__ partial, float* __restrict__ out, int B, int row) {
  __shared__ float part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (col < row)
    for (int bi = ty; bi < B; bi += 8) s += partial[static_cast<size_t>(bi) * row + col];
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < row) {
    float t = part[0][tx];
#pragma unroll
    for (int i = 1; i < 8; ++i) t += part[i][tx];
    out[col] = t;
  }
}

// ------------------------------------------------------------ log-space form
// MXK_LOGSPACE_FAST (default): exp / log through the special-function unit's approximations (ex2, lg2: relative
// error about 2^-22) instead of the full-precision library sequences, which are most of these kernels'
// instructions.  Measured against the fp64 oracle on the fused MinGRU path (8 x 256 x 256, inputs of a few units):
// x 8e-8, y 3e-7, cotangents 4e-7 / 6e-7 of each tensor's max-abs, against 8e-8, 2e-7, 2e-7 / 3e-7 with the library
// functions (-DMXK_LOGSPACE_FAST=0) -- both far inside the 1e-5 / 1e-4 the tests allow -- and 0.72 against 0.91 ms
// for the 256 x 256 x 1024 forward + backward.
#ifndef MXK_LOGSPACE_FAST
#define MXK_LOGSPACE_FAST 1
#endif
__device__ __forceinline__ float exp_ls(float x) { return MXK_LOGSPACE_FAST ? __expf(x) : expf(x); }
__device__ __forceinline__ float log_ls(float x) { return MXK_LOGSPACE_FAST ? __logf(x) : logf(x); }
// log(1 + e) for e in [0, 1]
__device__ __forceinline__ float log1p_ls(float e) { return MXK_LOGSPACE_FAST ? __logf(1.f + e) : log1pf(e); }

__device__ __forceinline__ float log_add_exp(float p, float q) {
  const float hi = fmaxf(p, q), lo = fminf(p, q);
  if (hi == -INFINITY) return -INFINITY;
  return hi + log1p_ls(exp_ls(lo - hi));
}

// MinGRU's gate math (min_gru.py:52-61), fused into the scan when the kernels are handed the Dense layers'
// pre-activations instead of the elements:
//   log_state = -softplus(-z) + log g(h~),  decay = -softplus(z),  g(h) = h >= 0 ? h + 0.5 : sigmoid(h).
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1p_ls(exp_ls(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + exp_ls(-x)); }
__device__ __forceinline__ float log_g(float h) { return h >= 0.f ? log_ls(h + 0.5f) : -softplus_f(-h); }
__device__ __forceinline__ float dlog_g(float h) { return h >= 0.f ? 1.f / (h + 0.5f) : sigmoid_f(-h); }

// GATES: `ls` / `d` hold the pre-activations z / h~ and the elements are formed on the fly.
template <int W, bool GATES>
__global__ void __launch_bounds__(kBlock)
loglinrec_fwd_kernel(const float* __restrict__ ls, const float* __restrict__ d,
                     const float* __restrict__ x0, const float* __restrict__ a0,
                     const uint8_t* __restrict__ done, float* __restrict__ x, float* __restrict__ y,
                     float* __restrict__ a_last, int B, int T, int row) {
  const int per_row = row / W;
  const long long gid = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  if (gid >= static_cast<long long>(B) * per_row) return;
  const int bi = static_cast<int>(gid / per_row);
  const int col = static_cast<int>(gid % per_row) * W;
  const size_t seq = static_cast<size_t>(bi) * T * row + col;
  const size_t crow = static_cast<size_t>(bi) * row + col;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  Pack<W> cur = x0 ? load_pack_cached<W>(x0 + crow) : fill_pack<W>(-INFINITY, 0.f, false);
  Pack<W> acc = (a_last && a0) ? load_pack_cached<W>(a0 + crow) : fill_pack<W>(0.f, 0.f, false);

  for (int t0 = 0; t0 < T; t0 += kUnroll) {
    Pack<W> lv[kUnroll], dv[kUnroll];
    unsigned flag[kUnroll];   // raw reset bytes: nothing in the load loop may wait for a loaded value
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = t0 + u;
      flag[u] = 0;
      if (t < T) {
        const size_t off = seq + static_cast<size_t>(t) * row;
        lv[u] = load_pack<W>(ls + off);
        dv[u] = load_pack<W>(d + off);
        if (drow) flag[u] = drow[t];
      }
    }
    bool rs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = t0 + u;
      rs[u] = flag[u] != 0;
      if (t < T) {
        Pack<W> yo;
#pragma unroll
        for (int i = 0; i < W; ++i) {
          if constexpr (GATES) {
            // softplus(z) = max(z, 0) + L and softplus(-z) = max(-z, 0) + L share L = log1p(exp(-|z|))
            const float z = lv[u].v[i], ht = dv[u].v[i];
            const float lz = log1p_ls(exp_ls(-fabsf(z)));
            lv[u].v[i] = log_g(ht) - (fmaxf(-z, 0.f) + lz);
            dv[u].v[i] = -(fmaxf(z, 0.f) + lz);
          }
          cur.v[i] = rs[u] ? lv[u].v[i] : log_add_exp(dv[u].v[i] + cur.v[i], lv[u].v[i]);
          acc.v[i] = rs[u] ? dv[u].v[i] : dv[u].v[i] + acc.v[i];
          yo.v[i] = exp_ls(cur.v[i]);
        }
        const size_t off = seq + static_cast<size_t>(t) * row;
        store_pack<W>(x + off, cur);
        if (y) store_pack<W>(y + off, yo);
      }
    }
  }
  if (a_last) {
#pragma unroll
    for (int i = 0; i < W; ++i) a_last[crow + i] = acc.v[i];
  }
}

// GATES: `d` holds z, `ht` the second pre-activation; gls / gd receive the cotangents of z / h~.
template <int W, bool GATES>
__global__ void __launch_bounds__(kBlock)
loglinrec_bwd_kernel(const float* __restrict__ d, const float* __restrict__ ht, const float* __restrict__ x,
                     const float* __restrict__ x0, const uint8_t* __restrict__ done,
                     const float* __restrict__ gx, const float* __restrict__ gy,
                     const float* __restrict__ gx_last, float* __restrict__ gls,
                     float* __restrict__ gd, float* __restrict__ gx0, int B, int T, int row) {
  const int per_row = row / W;
  const long long gid = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  if (gid >= static_cast<long long>(B) * per_row) return;
  const int bi = static_cast<int>(gid / per_row);
  const int col = static_cast<int>(gid % per_row) * W;
  const size_t seq = static_cast<size_t>(bi) * T * row + col;
  const size_t crow = static_cast<size_t>(bi) * row + col;
  const uint8_t* drow = done ? done + static_cast<size_t>(bi) * T : nullptr;

  // carry = w_{t+1} G_{t+1}
  Pack<W> carry = gx_last ? load_pack_cached<W>(gx_last + crow) : fill_pack<W>(0.f, 0.f, false);

  for (int t0 = T - 1; t0 >= 0; t0 -= kUnroll) {
    Pack<W> dv[kUnroll], xv[kUnroll], xp[kUnroll], gxv[kUnroll], gyv[kUnroll], hv[kUnroll];
    // The load loop issues every load of its steps without waiting for any: the decay and x_{t-1} are fetched
    // whether or not step t resets (a branch on the reset byte would hold the later loads back).
    unsigned flag[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = t0 - u;
      flag[u] = 0;
      if (t >= 0) {
        const size_t off = seq + static_cast<size_t>(t) * row;
        if (drow) flag[u] = drow[t];
        xv[u] = load_pack<W>(x + off);
        gxv[u] = gx ? load_pack<W>(gx + off) : fill_pack<W>(0.f, 0.f, false);
        if (gy) gyv[u] = load_pack<W>(gy + off);
        dv[u] = load_pack<W>(d + off);
        if constexpr (GATES) hv[u] = load_pack<W>(ht + off);
        if (t > 0) xp[u] = load_pack<W>(x + off - row);
        else xp[u] = x0 ? load_pack_cached<W>(x0 + crow) : fill_pack<W>(-INFINITY, 0.f, false);
      }
    }
    bool rs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int t = t0 - u;
      rs[u] = flag[u] != 0;
      if (t >= 0) {
        Pack<W> ols, od;
#pragma unroll
        for (int i = 0; i < W; ++i) {
          float g = gxv[u].v[i] + carry.v[i];
          if (gy) g = fmaf(gyv[u].v[i], exp_ls(xv[u].v[i]), g);
          float w = 0.f;
          float ez = 0.f;   // exp(-|z|): shared by softplus(z) here and sigmoid(z) below
          if constexpr (GATES) ez = exp_ls(-fabsf(dv[u].v[i]));
          if (!rs[u]) {
            const float dec = GATES ? -(fmaxf(dv[u].v[i], 0.f) + log1p_ls(ez)) : dv[u].v[i];
            const float p = dec + xp[u].v[i];
            w = (p == -INFINITY) ? 0.f : exp_ls(p - xv[u].v[i]);
          }
          od.v[i] = w * g;
          ols.v[i] = (1.f - w) * g;
          carry.v[i] = od.v[i];
          if constexpr (GATES) {
            // chain rule through the gate math: d(-softplus(-z))/dz = 1 - sigmoid(z), d(-softplus(z))/dz = -sigmoid(z)
            const float sg = (dv[u].v[i] >= 0.f ? 1.f : ez) / (1.f + ez);
            const float g_ls = ols.v[i], g_d = od.v[i];
            ols.v[i] = g_ls * (1.f - sg) - g_d * sg;
            od.v[i] = g_ls * dlog_g(hv[u].v[i]);
          }
        }
        const size_t off = seq + static_cast<size_t>(t) * row;
        store_pack<W>(gls + off, ols);
        store_pack<W>(gd + off, od);
      }
    }
  }
  if (gx0) {
#pragma unroll
    for (int i = 0; i < W; ++i) gx0[crow + i] = carry.v[i];
  }
}

// ------------------------------------------------------------- host helpers
// Wide packs when they give every SM at least two full blocks, else one
// element per thread (more, narrower threads keep more SMs busy on small B*D).
inline int pick_width(long long floats_total, int row, bool cplx, std::initializer_list<const void*> ptrs) {
  const int narrow = cplx ? 2 : 1;
  if (row % 4 != 0) return narrow;
  for (const void* p : ptrs)
    if (p && !aligned16(p)) return narrow;
  if (floats_total / 4 < 2LL * kNumSMs * kBlock) return narrow;
  return 4;
}

// Time-split kernels: narrow packs only (so few channels that wide packs would leave SMs idle),
// at most four blocks per SM of plain one-thread-per-channel work, and 32 <= T <= 256.
inline bool use_time_split(int w, long long floats_total, int T, bool cplx) {
  return w == (cplx ? 2 : 1) && floats_total <= 4LL * kNumSMs * kBlock && T >= 32 && T <= kSegs * 16;
}

inline unsigned blocks_for(long long threads) {
  return static_cast<unsigned>((threads + kBlock - 1) / kBlock);
}

inline int check_dims(int B, int T, int D) {
  if (B <= 0 || T <= 0 || D <= 0) return MXK_ERR_DIMS;
  if (static_cast<long long>(B) * D > (1LL << 40)) return MXK_ERR_DIMS;
  return MXK_OK;
}

template <bool CPLX>
int linrec_fwd(const float* a, int a_tinv, const float* b, const float* h0, const float* a0,
               const uint8_t* done, float* h, float* a_last, int B, int T, int D, mxk_stream_t stream) {
  if (!a || !b || !h) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  const int row = CPLX ? 2 * D : D;
  const int min_align = CPLX ? 8 : 4;
  for (const void* p : {(const void*)a, (const void*)b, (const void*)h0, (const void*)a0, (const void*)h, (const void*)a_last})
    if (p && (reinterpret_cast<uintptr_t>(p) % min_align)) return MXK_ERR_ALIGN;
  const long long total = static_cast<long long>(B) * row;
  const int w = pick_width(total, row, CPLX, {a, b, h0, a0, h, a_last});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // few channels, moderate T: split time too (one launch, T/16 sequential steps per thread)
  if (use_time_split(w, total, T, CPLX)) {
    const int len = (T + kSegs - 1) / kSegs;
    const unsigned threads = 32 * kSegs;
    if constexpr (CPLX) {
      const unsigned blocks = static_cast<unsigned>((total / 2 + 31) / 32);
      if (len <= 8) linrec_fwd_tsplit_kernel<true, 8, 2><<<blocks, threads, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
      else linrec_fwd_tsplit_kernel<true, 16, 2><<<blocks, threads, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
    } else {
      bool wide = (D % 4 == 0) && len <= 8;   // 16-byte lanes keep 8 steps x (a, b) in registers
      for (const void* ptr : {(const void*)a, (const void*)b, (const void*)h0, (const void*)a0, (const void*)h, (const void*)a_last})
        if (ptr && !aligned16(ptr)) wide = false;
      if (wide) {
        const unsigned blocks = static_cast<unsigned>((total / 4 + 31) / 32);
        linrec_fwd_tsplit_kernel<false, 8, 4><<<blocks, threads, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
      } else {
        const unsigned blocks = static_cast<unsigned>((total + 31) / 32);
        if (len <= 8) linrec_fwd_tsplit_kernel<false, 8, 1><<<blocks, threads, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
        else linrec_fwd_tsplit_kernel<false, 16, 1><<<blocks, threads, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
      }
    }
    return launch_status();
  }
  // A grid of at most three blocks per SM cannot cover the HBM latency with the default depth: such launches keep
  // two (16-byte packs) or four (narrow packs) times as many time steps of loads in flight, at half the occupancy.
  constexpr int kN = CPLX ? 2 : 1;
  const unsigned blocks = w == 4 ? blocks_for(total / 4) : blocks_for(total / kN);
  const bool small = blocks <= 3u * kNumSMs;
  if (w == 4) {
    if (small) linrec_fwd_kernel<CPLX, 4, 2 * MXK_LINREC_UNROLL_F, 2><<<blocks, kBlock, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
    else linrec_fwd_kernel<CPLX, 4><<<blocks, kBlock, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
  } else {
    if (small) linrec_fwd_kernel<CPLX, kN, 4 * MXK_LINREC_UNROLL_F, 2><<<blocks, kBlock, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
    else linrec_fwd_kernel<CPLX, kN><<<blocks, kBlock, 0, s>>>(a, a_tinv, b, h0, a0, done, h, a_last, B, T, row);
  }
  return launch_status();
}

// State after the last step only: one read stream, nothing stored per step (the deep-unroll variants:
// with no stores in flight the loads are all there is to overlap).
template <bool CPLX>
int linrec_last(const float* a, int a_tinv, const float* b, const float* h0, const uint8_t* done, float* h_last,
                int B, int T, int D, mxk_stream_t stream) {
  if (!a || !b || !h_last) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  const int row = CPLX ? 2 * D : D;
  const int min_align = CPLX ? 8 : 4;
  for (const void* p : {(const void*)a, (const void*)b, (const void*)h0, (const void*)h_last})
    if (p && (reinterpret_cast<uintptr_t>(p) % min_align)) return MXK_ERR_ALIGN;
  const long long total = static_cast<long long>(B) * row;
  const int w = pick_width(total, row, CPLX, {a, b, h0, h_last});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  constexpr int kN = CPLX ? 2 : 1;
  if (w == 4)
    linrec_fwd_kernel<CPLX, 4, 2 * MXK_LINREC_UNROLL_F, 2, true><<<blocks_for(total / 4), kBlock, 0, s>>>(
        a, a_tinv, b, h0, nullptr, done, h_last, nullptr, B, T, row);
  else
    linrec_fwd_kernel<CPLX, kN, 4 * MXK_LINREC_UNROLL_F, 2, true><<<blocks_for(total / kN), kBlock, 0, s>>>(
        a, a_tinv, b, h0, nullptr, done, h_last, nullptr, B, T, row);
  return launch_status();
}

template <bool CPLX>
int linrec_bwd(const float* a, int a_tinv, const float* h, const float* h0, const uint8_t* done,
               const float* gh, const float* gh_last, float* gb, float* ga, float* gh0,
               void* workspace, size_t workspace_bytes, int B, int T, int D, int conj_ops,
               mxk_stream_t stream) {
  if (!a || !h || !gh || !gb) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  const int row = CPLX ? 2 * D : D;
  const int min_align = CPLX ? 8 : 4;
  for (const void* p : {(const void*)a, (const void*)h, (const void*)h0, (const void*)gh, (const void*)gh_last,
                        (const void*)gb, (const void*)ga, (const void*)gh0, (const void*)workspace})
    if (p && (reinterpret_cast<uintptr_t>(p) % min_align)) return MXK_ERR_ALIGN;
  float* partial = nullptr;
  if (ga && a_tinv) {
    const size_t need = mxk_linrec_bwd_workspace_bytes(CPLX, 1, B, T, D);
    if (!workspace || workspace_bytes < need) return MXK_ERR_WORKSPACE;
    partial = static_cast<float*>(workspace);
  }
  const long long total = static_cast<long long>(B) * row;
  const int w = pick_width(total, row, CPLX, {a, h, h0, gh, gh_last, gb, ga, gh0, workspace});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ga_full = a_tinv ? nullptr : ga;
  if (use_time_split(w, total, T, CPLX)) {
    constexpr int kW = CPLX ? 2 : 1;
    const unsigned blocks = static_cast<unsigned>((total / kW + 31) / 32), threads = 32 * kSegs;
    if ((T + kSegs - 1) / kSegs <= 8)
      linrec_bwd_tsplit_kernel<CPLX, 8, kW><<<blocks, threads, 0, s>>>(a, a_tinv, h, h0, done, gh, gh_last, gb, ga_full, partial, gh0, B, T, row, conj_ops);
    else
      linrec_bwd_tsplit_kernel<CPLX, 16, kW><<<blocks, threads, 0, s>>>(a, a_tinv, h, h0, done, gh, gh_last, gb, ga_full, partial, gh0, B, T, row, conj_ops);
  } else {
    constexpr int kN = CPLX ? 2 : 1;
    const unsigned blocks = w == 4 ? blocks_for(total / 4) : blocks_for(total / kN);
    const bool small = blocks <= 3u * kNumSMs;   // see linrec_fwd
    if (w == 4) {
      if (small) linrec_bwd_kernel<CPLX, 4, 2 * MXK_LINREC_UNROLL_B, 2><<<blocks, kBlock, 0, s>>>(a, a_tinv, h, h0, done, gh, gh_last, gb, ga_full, partial, gh0, B, T, row, conj_ops);
      else linrec_bwd_kernel<CPLX, 4><<<blocks, kBlock, 0, s>>>(a, a_tinv, h, h0, done, gh, gh_last, gb, ga_full, partial, gh0, B, T, row, conj_ops);
    } else {
      if (small) linrec_bwd_kernel<CPLX, kN, 4 * MXK_LINREC_UNROLL_B, 2><<<blocks, kBlock, 0, s>>>(a, a_tinv, h, h0, done, gh, gh_last, gb, ga_full, partial, gh0, B, T, row, conj_ops);
      else linrec_bwd_kernel<CPLX, kN><<<blocks, kBlock, 0, s>>>(a, a_tinv, h, h0, done, gh, gh_last, gb, ga_full, partial, gh0, B, T, row, conj_ops);
    }
  }
  if (int st = launch_status()) return st;
  if (partial) {
    reduce_rows_kernel<<<(row + 31) / 32, kBlock, 0, s>>>(partial, ga, B, row);
    return launch_status();
  }
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

// ---------------------------------------------------------------------------
// Built-in scratch for mxk_linrec_c64_bwd_noalloc: one fixed array per GPU that
// loads this library, resident until the process exits.
// ---------------------------------------------------------------------------
namespace mxk {
namespace {

constexpr size_t kNoAllocScratchFloats = 1u << 20;  // 4 MiB: B * D <= 524288 complex elements
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_ptr[kMaxDevices] = {};

// Device address of g_noalloc_scratch on the current device.  In host code the
// symbol itself is only a handle, so the address is looked up once per device
// (with that device current) and cached.
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return MXK_ERR_DIMS;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_noalloc_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_noalloc_ptr[dev];
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

extern "C" {

int mxk_linrec_f32_fwd(const float* a, int a_time_invariant, const float* b, const float* h0,
                       const float* a0, const uint8_t* done, float* h, float* a_last,
                       int B, int T, int D, mxk_stream_t stream) {
  return mxk::linrec_fwd<false>(a, a_time_invariant, b, h0, a0, done, h, a_last, B, T, D, stream);
}

int mxk_linrec_c64_fwd(const float* a, int a_time_invariant, const float* b, const float* h0,
                       const float* a0, const uint8_t* done, float* h, float* a_last,
                       int B, int T, int D, mxk_stream_t stream) {
  return mxk::linrec_fwd<true>(a, a_time_invariant, b, h0, a0, done, h, a_last, B, T, D, stream);
}

int mxk_linrec_f32_last(const float* a, int a_time_invariant, const float* b, const float* h0, const uint8_t* done,
                        float* h_last, int B, int T, int D, mxk_stream_t stream) {
  return mxk::linrec_last<false>(a, a_time_invariant, b, h0, done, h_last, B, T, D, stream);
}

int mxk_linrec_c64_last(const float* a, int a_time_invariant, const float* b, const float* h0, const uint8_t* done,
                        float* h_last, int B, int T, int D, mxk_stream_t stream) {
  return mxk::linrec_last<true>(a, a_time_invariant, b, h0, done, h_last, B, T, D, stream);
}

size_t mxk_linrec_bwd_workspace_bytes(int is_complex, int a_time_invariant, int B, int T, int D) {
  (void)T;
  if (!a_time_invariant || B <= 0 || D <= 0) return 0;
  return static_cast<size_t>(B) * D * (is_complex ? 2 : 1) * sizeof(float);
}

int mxk_linrec_f32_bwd(const float* a, int a_time_invariant, const float* h, const float* h0,
                       const uint8_t* done, const float* gh, const float* gh_last, float* gb,
                       float* ga, float* gh0, void* workspace, size_t workspace_bytes,
                       int B, int T, int D, mxk_stream_t stream) {
  return mxk::linrec_bwd<false>(a, a_time_invariant, h, h0, done, gh, gh_last, gb, ga, gh0, workspace,
                                workspace_bytes, B, T, D, 0, stream);
}

int mxk_linrec_c64_bwd(const float* a, int a_time_invariant, const float* h, const float* h0,
                       const uint8_t* done, const float* gh, const float* gh_last, float* gb,
                       float* ga, float* gh0, void* workspace, size_t workspace_bytes,
                       int B, int T, int D, int conjugate, mxk_stream_t stream) {
  return mxk::linrec_bwd<true>(a, a_time_invariant, h, h0, done, gh, gh_last, gb, ga, gh0, workspace,
                               workspace_bytes, B, T, D, conjugate, stream);
}

size_t mxk_linrec_noalloc_max_elements(void) { return mxk::kNoAllocScratchFloats / 2; }

int mxk_linrec_c64_bwd_noalloc(const float* a, const float* h, const float* h0, const uint8_t* done,
                               const float* gh, const float* gh_last, float* gb, float* ga, float* gh0,
                               int B, int T, int D, int conjugate, mxk_stream_t stream) {
  if (B <= 0 || T <= 0 || D <= 0) return MXK_ERR_DIMS;
  if (static_cast<size_t>(B) * static_cast<size_t>(D) > mxk_linrec_noalloc_max_elements()) return MXK_ERR_SCRATCH_LIMIT;
  float* scratch = nullptr;
  if (int st = mxk::noalloc_scratch(&scratch)) return st;
  return mxk::linrec_bwd<true>(a, /*a_tinv=*/1, h, h0, done, gh, gh_last, gb, ga, gh0, scratch,
                               mxk::kNoAllocScratchFloats * sizeof(float), B, T, D, conjugate, stream);
}

int mxk_loglinrec_f32_fwd(const float* ls, const float* d, const float* x0, const float* a0,
                          const uint8_t* done, float* x, float* y, float* a_last,
                          int B, int T, int D, mxk_stream_t stream) {
  using namespace mxk;
  if (!ls || !d || !x) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  for (const void* p : {(const void*)ls, (const void*)d, (const void*)x0, (const void*)a0, (const void*)x, (const void*)y, (const void*)a_last})
    if (p && (reinterpret_cast<uintptr_t>(p) % 4)) return MXK_ERR_ALIGN;
  const long long total = static_cast<long long>(B) * D;
  const int w = pick_width(total, D, false, {ls, d, x0, a0, x, y, a_last});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w == 4)
    loglinrec_fwd_kernel<4, false><<<blocks_for(total / 4), kBlock, 0, s>>>(ls, d, x0, a0, done, x, y, a_last, B, T, D);
  else
    loglinrec_fwd_kernel<1, false><<<blocks_for(total), kBlock, 0, s>>>(ls, d, x0, a0, done, x, y, a_last, B, T, D);
  return launch_status();
}

int mxk_mingru_f32_fwd(const float* z, const float* h_tilde, const float* x0, const float* a0, const uint8_t* done,
                       float* x, float* y, float* a_last, int B, int T, int D, mxk_stream_t stream) {
  using namespace mxk;
  if (!z || !h_tilde || !x) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  for (const void* p : {(const void*)z, (const void*)h_tilde, (const void*)x0, (const void*)a0, (const void*)x, (const void*)y, (const void*)a_last})
    if (p && (reinterpret_cast<uintptr_t>(p) % 4)) return MXK_ERR_ALIGN;
  const long long total = static_cast<long long>(B) * D;
  const int w = pick_width(total, D, false, {z, h_tilde, x0, a0, x, y, a_last});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w == 4)
    loglinrec_fwd_kernel<4, true><<<blocks_for(total / 4), kBlock, 0, s>>>(z, h_tilde, x0, a0, done, x, y, a_last, B, T, D);
  else
    loglinrec_fwd_kernel<1, true><<<blocks_for(total), kBlock, 0, s>>>(z, h_tilde, x0, a0, done, x, y, a_last, B, T, D);
  return launch_status();
}

int mxk_loglinrec_f32_bwd(const float* d, const float* x, const float* x0, const uint8_t* done,
                          const float* gx, const float* gy, const float* gx_last, float* gls,
                          float* gd, float* gx0, int B, int T, int D, mxk_stream_t stream) {
  using namespace mxk;
  if (!d || !x || !gls || !gd || (!gx && !gy)) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  for (const void* p : {(const void*)d, (const void*)x, (const void*)x0, (const void*)gx, (const void*)gy,
                        (const void*)gx_last, (const void*)gls, (const void*)gd, (const void*)gx0})
    if (p && (reinterpret_cast<uintptr_t>(p) % 4)) return MXK_ERR_ALIGN;
  const long long total = static_cast<long long>(B) * D;
  const int w = pick_width(total, D, false, {d, x, x0, gx, gy, gx_last, gls, gd, gx0});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w == 4)
    loglinrec_bwd_kernel<4, false><<<blocks_for(total / 4), kBlock, 0, s>>>(d, nullptr, x, x0, done, gx, gy, gx_last, gls, gd, gx0, B, T, D);
  else
    loglinrec_bwd_kernel<1, false><<<blocks_for(total), kBlock, 0, s>>>(d, nullptr, x, x0, done, gx, gy, gx_last, gls, gd, gx0, B, T, D);
  return launch_status();
}

int mxk_mingru_f32_bwd(const float* z, const float* h_tilde, const float* x, const float* x0, const uint8_t* done,
                       const float* gx, const float* gy, const float* gx_last, float* gz, float* gh, float* gx0,
                       int B, int T, int D, mxk_stream_t stream) {
  using namespace mxk;
  if (!z || !h_tilde || !x || !gz || !gh || (!gx && !gy)) return MXK_ERR_NULL;
  if (int st = check_dims(B, T, D)) return st;
  for (const void* p : {(const void*)z, (const void*)h_tilde, (const void*)x, (const void*)x0, (const void*)gx, (const void*)gy,
                        (const void*)gx_last, (const void*)gz, (const void*)gh, (const void*)gx0})
    if (p && (reinterpret_cast<uintptr_t>(p) % 4)) return MXK_ERR_ALIGN;
  const long long total = static_cast<long long>(B) * D;
  const int w = pick_width(total, D, false, {z, h_tilde, x, x0, gx, gy, gx_last, gz, gh, gx0});
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w == 4)
    loglinrec_bwd_kernel<4, true><<<blocks_for(total / 4), kBlock, 0, s>>>(z, h_tilde, x, x0, done, gx, gy, gx_last, gz, gh, gx0, B, T, D);
  else
    loglinrec_bwd_kernel<1, true><<<blocks_for(total), kBlock, 0, s>>>(z, h_tilde, x, x0, done, gx, gy, gx_last, gz, gh, gx0, B, T, D);
  return launch_status();
}

}  // extern "C"
