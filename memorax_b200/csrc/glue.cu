// Row-wise glue around the mixers, fused into single bandwidth-bound passes (bf16 in / out, fp32 math):
//   - LayerNorm / RMSNorm forward and backward (PreNorm's LayerNorm, blocks/normalization.py:10-35; the
//     RMSNorm in front of the cells' output projection, linear_attention.py:114),
//   - the gated residual y = x + sigmoid(g) * o and its backward (blocks/residual.py:53-59),
//   - per-head L2 normalisation of q / k and its backward (the delta-rule cell's key / query normalisation).
// One warp owns one row of D <= 1024 elements (D a multiple of 256): each lane holds D / 32 of them as 16-byte
// vectors, statistics are warp reductions, nothing goes through shared memory.  The (D,) parameter gradients
// are accumulated per warp in registers over a grid-stride loop of rows, combined per block in shared memory
// and written as one partial row per block; a second kernel adds the blocks in index order (no atomics:
// bit-reproducible).
#include <cuda_bf16.h>

#include "mxk_common.cuh"
#include "umma.cuh"

namespace mxk {
namespace {

constexpr int kRowWarps = 8;   // warps (rows in flight) per block

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

// V = D / 256 16-byte vectors per lane; lane l owns elements [v * 256 + l * 8, + 8).
template <int V>
__device__ __forceinline__ void load_row(const __nv_bfloat16* row, int lane, float (*x)[8]) {
#pragma unroll
  for (int v = 0; v < V; ++v) umma::unpack8_bf16(*reinterpret_cast<const uint4*>(row + v * 256 + lane * 8), x[v]);
}
template <int V>
__device__ __forceinline__ void store_row(__nv_bfloat16* row, int lane, const float (*y)[8]) {
#pragma unroll
  for (int v = 0; v < V; ++v) *reinterpret_cast<uint4*>(row + v * 256 + lane * 8) = umma::pack8_bf16(y[v]);
}

template <int V, bool RMS>
__global__ void __launch_bounds__(kRowWarps * 32)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                float* __restrict__ rstd, long long rows, float eps) {
  constexpr int D = V * 256;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float g[V][8], b[V][8];
  load_row<V>(gamma, lane, g);
  if (!RMS && beta) load_row<V>(beta, lane, b);
  for (long long r = static_cast<long long>(blockIdx.x) * kRowWarps + warp; r < rows; r += static_cast<long long>(gridDim.x) * kRowWarps) {
    float xv[V][8];
    load_row<V>(x + r * D, lane, xv);
    float s = 0.f;
    if (!RMS) {
#pragma unroll
      for (int v = 0; v < V; ++v)
#pragma unroll
        for (int e = 0; e < 8; ++e) s += xv[v][e];
      s = warp_sum(s) * (1.f / D);
    }
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) { const float c = xv[v][e] - s; q = fmaf(c, c, q); }
    const float rs = rsqrtf(warp_sum(q) * (1.f / D) + eps);
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float h = (xv[v][e] - s) * rs * g[v][e];
        xv[v][e] = (!RMS && beta) ? h + b[v][e] : h;
      }
    store_row<V>(y + r * D, lane, xv);
    if (lane == 0) {
      if (mean) mean[r] = s;
      rstd[r] = rs;
    }
  }
}

// dx per row; per-block partial sums of dgamma (and dbeta) into part[block][2][D].
template <int V, bool RMS>
__global__ void __launch_bounds__(kRowWarps * 32)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ part, long long rows) {
  constexpr int D = V * 256;
  __shared__ float red[kRowWarps][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float g[V][8], dg[V][8], db[V][8];
  load_row<V>(gamma, lane, g);
#pragma unroll
  for (int v = 0; v < V; ++v)
#pragma unroll
    for (int e = 0; e < 8; ++e) dg[v][e] = db[v][e] = 0.f;
  for (long long r = static_cast<long long>(blockIdx.x) * kRowWarps + warp; r < rows; r += static_cast<long long>(gridDim.x) * kRowWarps) {
    float xv[V][8], dv[V][8];
    load_row<V>(x + r * D, lane, xv);
    load_row<V>(dy + r * D, lane, dv);
    const float mu = RMS ? 0.f : mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = (xv[v][e] - mu) * rs, gy = dv[v][e] * g[v][e];
        dg[v][e] = fmaf(dv[v][e], xh, dg[v][e]);
        db[v][e] += dv[v][e];
        xv[v][e] = xh;
        dv[v][e] = gy;
        s1 += gy;
        s2 = fmaf(gy, xh, s2);
      }
    s1 = RMS ? 0.f : warp_sum(s1) * (1.f / D);
    s2 = warp_sum(s2) * (1.f / D);
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) xv[v][e] = rs * (dv[v][e] - s1 - xv[v][e] * s2);
    store_row<V>(dx + r * D, lane, xv);
  }
  // block partials: the eight warps' sums added in warp order
  for (int pass = 0; pass < (RMS ? 1 : 2); ++pass) {
    __syncthreads();
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) red[warp][v * 256 + lane * 8 + e] = pass == 0 ? dg[v][e] : db[v][e];
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += kRowWarps * 32) {
      float s = red[0][c];
#pragma unroll
      for (int w = 1; w < kRowWarps; ++w) s += red[w][c];
      part[(static_cast<size_t>(blockIdx.x) * 2 + pass) * D + c] = s;
    }
  }
}

// Adds the per-block partial rows in a fixed order: a block owns 32 columns, its eight thread rows each add
// every eighth partial, then thread row 0 adds the eight sums in order.
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(const float* __restrict__ part, float* __restrict__ dgamma, float* __restrict__ dbeta, int blocks, int D) {
  __shared__ float red[2][8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float sg = 0.f, sb = 0.f;
  if (c < D) {
    for (int b = ty; b < blocks; b += 8) {
      sg += part[(static_cast<size_t>(b) * 2) * D + c];
      if (dbeta) sb += part[(static_cast<size_t>(b) * 2 + 1) * D + c];
    }
  }
  red[0][ty][tx] = sg;
  red[1][ty][tx] = sb;
  __syncthreads();
  if (ty == 0 && c < D) {
    float tg = red[0][0][tx], tb = red[1][0][tx];
#pragma unroll
    for (int i = 1; i < 8; ++i) { tg += red[0][i][tx]; tb += red[1][i][tx]; }
    dgamma[c] = tg;
    if (dbeta) dbeta[c] = tb;
  }
}

// Column sums of a (rows, cols) bf16 matrix in fp32 -- the bias gradient of a Dense layer.  Block (cx, ry) owns 256
// columns x a contiguous range of rows: its thread (tx, ty) adds 8 columns of every eighth row, the eight thread rows
// are added in a fixed order, and the block's sums go to part[ry][col]; the second kernel adds the row blocks in order.
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const uint4* __restrict__ x, float* __restrict__ part, long long rows, int cols8, int rows_per_block) {
  __shared__ float red[8][32][9];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int v = blockIdx.x * 32 + tx;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  if (v < cols8) {
    long long r = r0 + ty;
    for (; r + 56 < r1; r += 64) {   // eight independent loads in flight
      uint4 raw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) raw[u] = ld_stream(x + (r + 8 * u) * cols8 + v);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float f[8];
        umma::unpack8_bf16(raw[u], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
    }
    for (; r < r1; r += 8) {
      float f[8];
      umma::unpack8_bf16(ld_stream(x + r * cols8 + v), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[ty][tx][e] = acc[e];
  __syncthreads();
  // 256 threads = 32 vectors x 8 elements: thread (tx2, e) adds the eight thread rows in order
  const int e = threadIdx.x & 7, tx2 = threadIdx.x >> 3;
  const int col = (blockIdx.x * 32 + tx2) * 8 + e;
  if (col < cols8 * 8) {
    float t = red[0][tx2][e];
#pragma unroll
    for (int i = 1; i < 8; ++i) t += red[i][tx2][e];
    part[static_cast<size_t>(blockIdx.y) * cols8 * 8 + col] = t;
  }
}
// A block owns 32 columns; its eight thread rows each add every eighth row block, then thread row 0 adds the eight sums in order.
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int row_blocks, int cols) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float t = 0.f;
  if (c < cols)
    for (int b = ty; b < row_blocks; b += 8) t += part[static_cast<size_t>(b) * cols + c];
  red[ty][tx] = t;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float u = red[0][tx];
#pragma unroll
    for (int i = 1; i < 8; ++i) u += red[i][tx];
    out[c] = __float2bfloat16(u);
  }
}

// GELU in its tanh form (flax's nn.gelu default, blocks/ffn.py:16): y = x/2 (1 + tanh(c (x + 0.044715 x^3))), c = sqrt(2/pi).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__global__ void __launch_bounds__(256)
gelu_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long n8) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n8) return;
  float f[8];
  umma::unpack8_bf16(ld_stream(x + i), f);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float v = f[e];
    const float t = tanh_fast(0.7978845608f * fmaf(0.044715f * v, v * v, v));
    f[e] = 0.5f * v * (1.f + t);
  }
  y[i] = umma::pack8_bf16(f);
}
// dx = dy * d/dx gelu(x)
__global__ void __launch_bounds__(256)
gelu_bwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, uint4* __restrict__ dx, long long n8) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n8) return;
  float f[8], g[8];
  umma::unpack8_bf16(ld_stream(x + i), f);
  umma::unpack8_bf16(ld_stream(dy + i), g);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float v = f[e], v2 = v * v;
    const float t = tanh_fast(0.7978845608f * fmaf(0.044715f * v, v2, v));
    const float dt = (1.f - t * t) * 0.7978845608f * fmaf(3.f * 0.044715f, v2, 1.f);
    g[e] *= 0.5f * (1.f + t) + 0.5f * v * dt;
  }
  dx[i] = umma::pack8_bf16(g);
}

// y = x + sigmoid(g) * o
__global__ void __launch_bounds__(256)
gated_residual_fwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ g, const uint4* __restrict__ o,
                          uint4* __restrict__ y, long long n8) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n8) return;
  float xf[8], gf[8], of[8];
  umma::unpack8_bf16(x[i], xf);
  umma::unpack8_bf16(g[i], gf);
  umma::unpack8_bf16(o[i], of);
#pragma unroll
  for (int e = 0; e < 8; ++e) xf[e] = fmaf(1.f / (1.f + __expf(-gf[e])), of[e], xf[e]);
  y[i] = umma::pack8_bf16(xf);
}
// do = dy * sigmoid(g), dg = dy * o * sigmoid(g) (1 - sigmoid(g)); dx = dy needs no kernel
__global__ void __launch_bounds__(256)
gated_residual_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ g, const uint4* __restrict__ o,
                          uint4* __restrict__ dg, uint4* __restrict__ d_o, long long n8) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n8) return;
  float yf[8], gf[8], of[8];
  umma::unpack8_bf16(dy[i], yf);
  umma::unpack8_bf16(g[i], gf);
  umma::unpack8_bf16(o[i], of);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float s = 1.f / (1.f + __expf(-gf[e]));
    gf[e] = yf[e] * of[e] * s * (1.f - s);
    of[e] = yf[e] * s;
  }
  dg[i] = umma::pack8_bf16(gf);
  d_o[i] = umma::pack8_bf16(of);
}

// Per-head L2 normalisation: LPH = hd / 8 lanes hold one head vector (16 bytes each).
template <int LPH, bool BWD>
__global__ void __launch_bounds__(256)
l2norm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy, uint4* __restrict__ out, long long nvec, float eps) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const bool in = i < nvec;
  float xf[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, df[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (in) {
    umma::unpack8_bf16(x[i], xf);
    if (BWD) umma::unpack8_bf16(dy[i], df);
  }
  float ss = 0.f, sd = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) { ss = fmaf(xf[e], xf[e], ss); sd = fmaf(xf[e], df[e], sd); }
#pragma unroll
  for (int off = 1; off < LPH; off <<= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (BWD) sd += __shfl_xor_sync(0xffffffffu, sd, off);
  }
  const float inv = 1.f / fmaxf(sqrtf(ss), eps);
  if (BWD) {
    // y = x inv;  dx = inv (dy - y (y . dy))
    const float ydy = sd * inv;
#pragma unroll
    for (int e = 0; e < 8; ++e) xf[e] = inv * (df[e] - xf[e] * inv * ydy);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) xf[e] *= inv;
  }
  if (in) out[i] = umma::pack8_bf16(xf);
}

int check_norm(const void* x, const void* gamma, const void* y, long long rows, int D) {
  if (!x || !gamma || !y) return MXK_ERR_NULL;
  if (rows <= 0 || D <= 0) return MXK_ERR_DIMS;
  if (D % 256 != 0 || D > 1024) return MXK_ERR_UNSUPPORTED;
  for (const void* p : {x, gamma, y})
    if (!aligned16(p)) return MXK_ERR_ALIGN;
  return MXK_OK;
}

// Blocks of the backward row pass: two per SM -- enough rows per warp to amortise the partial row every
// block writes, few enough partials for the fixed-order reduction.  The forward pass takes eight per SM.
int norm_blocks(long long rows, int per_sm = 2) {
  const long long want = (rows + kRowWarps - 1) / kRowWarps;
  const long long cap = static_cast<long long>(per_sm) * kNumSMs;
  return static_cast<int>(want < cap ? want : cap);
}

// Row blocks of the column-sum kernels: about four blocks per SM over all column strips, at least 32 rows each.
int colsum_row_blocks(long long rows, int cols) {
  const int strips = (cols / 8 + 31) / 32;
  long long want = (4LL * kNumSMs + strips - 1) / strips;
  const long long most = (rows + 31) / 32;
  if (want > most) want = most;
  if (want > 512) want = 512;
  return static_cast<int>(want < 1 ? 1 : want);
}

}  // namespace
}  // namespace mxk

extern "C" {

size_t mxk_colsum_workspace_bytes(long long rows, int cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>(mxk::colsum_row_blocks(rows, cols)) * cols * sizeof(float);
}

int mxk_colsum_bf16(const void* x, void* out, void* workspace, size_t workspace_bytes, long long rows, int cols,
                    mxk_stream_t stream) {
  using namespace mxk;
  if (!x || !out) return MXK_ERR_NULL;
  if (rows <= 0 || cols <= 0) return MXK_ERR_DIMS;
  if (cols % 8) return MXK_ERR_UNSUPPORTED;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(out) % 2) || (workspace && !aligned16(workspace))) return MXK_ERR_ALIGN;
  if (!workspace || workspace_bytes < mxk_colsum_workspace_bytes(rows, cols)) return MXK_ERR_WORKSPACE;
  const int nrb = colsum_row_blocks(rows, cols), cols8 = cols / 8;
  const int rpb = static_cast<int>((rows + nrb - 1) / nrb);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  colsum_partial_kernel<<<dim3((cols8 + 31) / 32, nrb), 256, 0, s>>>(static_cast<const uint4*>(x), static_cast<float*>(workspace),
                                                                      rows, cols8, rpb);
  if (int st = launch_status()) return st;
  colsum_final_kernel<<<(cols + 31) / 32, 256, 0, s>>>(static_cast<const float*>(workspace), static_cast<__nv_bfloat16*>(out), nrb, cols);
  return launch_status();
}

size_t mxk_norm_bwd_workspace_bytes(long long rows, int D) {
  if (rows <= 0 || D <= 0) return 0;
  return static_cast<size_t>(mxk::norm_blocks(rows)) * 2 * D * sizeof(float);
}

int mxk_norm_bf16_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                      long long rows, int D, float eps, int rms, mxk_stream_t stream) {
  using namespace mxk;
  if (int st = check_norm(x, gamma, y, rows, D)) return st;
  if (!rstd || (!rms && !mean)) return MXK_ERR_NULL;
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* gp = static_cast<const __nv_bfloat16*>(gamma);
  const auto* bp = static_cast<const __nv_bfloat16*>(beta);
  auto* yp = static_cast<__nv_bfloat16*>(y);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = norm_blocks(rows, 8), threads = kRowWarps * 32;
#define MXK_NORM_FWD(V)                                                                                        \
  if (rms) norm_fwd_kernel<V, true><<<blocks, threads, 0, s>>>(xp, gp, nullptr, yp, nullptr, rstd, rows, eps); \
  else norm_fwd_kernel<V, false><<<blocks, threads, 0, s>>>(xp, gp, bp, yp, mean, rstd, rows, eps);
  switch (D / 256) {
    case 1: MXK_NORM_FWD(1) break;
    case 2: MXK_NORM_FWD(2) break;
    case 3: MXK_NORM_FWD(3) break;
    default: MXK_NORM_FWD(4) break;
  }
#undef MXK_NORM_FWD
  return launch_status();
}

int mxk_norm_bf16_bwd(const void* x, const void* gamma, const float* mean, const float* rstd, const void* dy, void* dx,
                      float* dgamma, float* dbeta, void* workspace, size_t workspace_bytes, long long rows, int D, int rms,
                      mxk_stream_t stream) {
  using namespace mxk;
  if (int st = check_norm(x, gamma, dx, rows, D)) return st;
  if (!rstd || !dy || !dgamma || (!rms && (!mean || !dbeta))) return MXK_ERR_NULL;
  if (!workspace || workspace_bytes < mxk_norm_bwd_workspace_bytes(rows, D)) return MXK_ERR_WORKSPACE;
  if (!aligned16(dy) || (reinterpret_cast<uintptr_t>(workspace) & 3u)) return MXK_ERR_ALIGN;
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* gp = static_cast<const __nv_bfloat16*>(gamma);
  const auto* dyp = static_cast<const __nv_bfloat16*>(dy);
  auto* dxp = static_cast<__nv_bfloat16*>(dx);
  float* part = static_cast<float*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = norm_blocks(rows), threads = kRowWarps * 32;
#define MXK_NORM_BWD(V)                                                                                  \
  if (rms) norm_bwd_kernel<V, true><<<blocks, threads, 0, s>>>(xp, gp, nullptr, rstd, dyp, dxp, part, rows); \
  else norm_bwd_kernel<V, false><<<blocks, threads, 0, s>>>(xp, gp, mean, rstd, dyp, dxp, part, rows);
  switch (D / 256) {
    case 1: MXK_NORM_BWD(1) break;
    case 2: MXK_NORM_BWD(2) break;
    case 3: MXK_NORM_BWD(3) break;
    default: MXK_NORM_BWD(4) break;
  }
#undef MXK_NORM_BWD
  if (int st = launch_status()) return st;
  norm_bwd_reduce_kernel<<<(D + 31) / 32, 256, 0, s>>>(part, dgamma, rms ? nullptr : dbeta, blocks, D);
  return launch_status();
}

int mxk_gelu_bf16(const void* x, const void* dy, void* out, long long n, mxk_stream_t stream) {
  using namespace mxk;
  if (!x || !out) return MXK_ERR_NULL;
  if (n <= 0 || n % 8) return MXK_ERR_DIMS;
  for (const void* p : {x, dy, (const void*)out})
    if (p && !aligned16(p)) return MXK_ERR_ALIGN;
  const long long n8 = n / 8;
  const unsigned blocks = static_cast<unsigned>((n8 + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dy) gelu_bwd_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(dy), static_cast<uint4*>(out), n8);
  else gelu_fwd_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint4*>(x), static_cast<uint4*>(out), n8);
  return launch_status();
}

int mxk_gated_residual_bf16_fwd(const void* x, const void* g, const void* o, void* y, long long n, mxk_stream_t stream) {
  using namespace mxk;
  if (!x || !g || !o || !y) return MXK_ERR_NULL;
  if (n <= 0 || n % 8) return MXK_ERR_DIMS;
  for (const void* p : {x, g, o, (const void*)y})
    if (!aligned16(p)) return MXK_ERR_ALIGN;
  const long long n8 = n / 8;
  gated_residual_fwd_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(g), static_cast<const uint4*>(o), static_cast<uint4*>(y), n8);
  return launch_status();
}

int mxk_gated_residual_bf16_bwd(const void* dy, const void* g, const void* o, void* dg, void* d_o, long long n,
                                mxk_stream_t stream) {
  using namespace mxk;
  if (!dy || !g || !o || !dg || !d_o) return MXK_ERR_NULL;
  if (n <= 0 || n % 8) return MXK_ERR_DIMS;
  for (const void* p : {dy, g, o, (const void*)dg, (const void*)d_o})
    if (!aligned16(p)) return MXK_ERR_ALIGN;
  const long long n8 = n / 8;
  gated_residual_bwd_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(dy), static_cast<const uint4*>(g), static_cast<const uint4*>(o), static_cast<uint4*>(dg),
      static_cast<uint4*>(d_o), n8);
  return launch_status();
}

int mxk_l2norm_heads_bf16(const void* x, const void* dy, void* out, long long vectors, int head_dim, float eps,
                          mxk_stream_t stream) {
  using namespace mxk;
  if (!x || !out) return MXK_ERR_NULL;
  if (vectors <= 0) return MXK_ERR_DIMS;
  if (head_dim != 64 && head_dim != 128) return MXK_ERR_UNSUPPORTED;
  for (const void* p : {x, dy, (const void*)out})
    if (p && !aligned16(p)) return MXK_ERR_ALIGN;
  const long long nvec = vectors * (head_dim / 8);
  const unsigned blocks = static_cast<unsigned>((nvec + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* xp = static_cast<const uint4*>(x);
  const uint4* dp = static_cast<const uint4*>(dy);
  uint4* op = static_cast<uint4*>(out);
  if (head_dim == 64) {
    if (dy) l2norm_kernel<8, true><<<blocks, 256, 0, s>>>(xp, dp, op, nvec, eps);
    else l2norm_kernel<8, false><<<blocks, 256, 0, s>>>(xp, nullptr, op, nvec, eps);
  } else {
    if (dy) l2norm_kernel<16, true><<<blocks, 256, 0, s>>>(xp, dp, op, nvec, eps);
    else l2norm_kernel<16, false><<<blocks, 256, 0, s>>>(xp, nullptr, op, nvec, eps);
  }
  return launch_status();
}

}  // extern "C"
