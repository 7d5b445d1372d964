// Thin inline-PTX layer over the sm_100a tensor-core path: tcgen05.mma with
// shared-memory operand descriptors, TMEM allocation and access, mbarrier
// completion with bounded waits.
//
// Shared-memory operand format used throughout ("panels"): a matrix X[r][c] of
// 2-byte elements is stored as [c / 8][r][c % 8], i.e. 16-byte vectors of eight
// consecutive c, all rows of a vector column contiguous.  Without swizzling this
// one format is both canonical layouts tcgen05 accepts:
//   - contraction over c ("K-major"):  LBO = rows * 16 (next 8 c), SBO = 128
//     (next 8 rows); one K=16 instruction spans two panels, so the K loop
//     advances the start address by 2 * rows * 16 bytes;
//   - contraction over r ("MN-major"): SBO = rows * 16 (next 8 c), LBO = 128
//     (next 8 rows); the K loop advances by 16 rows = 256 bytes.
// A thread that owns row r writes eight consecutive c with one 16-byte store.
//
// Accumulators of M = 64 instructions (cta_group::1) live in TMEM lanes
// 32 * (row / 16) + row % 16, so warp w of a 128-thread CTA reads rows
// 16 w .. 16 w + 15 with its lanes 0..15 (tcgen05.ld.32x32b); lanes 16..31 of
// every warp see unused TMEM lanes.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace mxk {
namespace umma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- descriptors -----------------------------------------------------------
// 64-bit shared-memory matrix descriptor, no swizzle, Blackwell version bit set.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// 32-bit instruction descriptor for kind::f16 with bf16 operands, fp32 accumulate.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// 128-byte-swizzled row-major tiles ("SW tiles"): rows of 64 two-byte elements, one 128-byte line per
// row, the 16-byte chunk j of row r stored at chunk position j ^ (r & 7); tile base 1024-byte aligned.
// This is what a tiled TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes (128-byte pieces instead of the
// panel format's 16-byte pieces), and it is again both canonical tcgen05 layouts:
//   - contraction over the columns (K-major): SBO = 1024 (next 8 rows), 32 bytes per K = 16 step;
//   - contraction over the rows (MN-major): SBO = 1024 (next 8 rows), 2048 bytes per K = 16 step,
//     LBO = distance to the next 64-column block when M or N exceeds 64.
// Validated on the device against a CPU GEMM for both majors, M = 64 / 128, N = 32..128.
__device__ __forceinline__ int sw_idx(int r, int chunk) { return r * 8 + (chunk ^ (r & 7)); }   // uint4 index

// Operand in panel format with `rows` rows, or (swizzled) an SW tile; `contract_rows` selects which
// index is the contraction (K) index of the MMA.
struct Operand {
  uint32_t saddr;
  uint32_t rows;
  bool contract_rows;
  bool swizzled = false;
  uint32_t block_stride = 16;   // SW tiles, contraction over rows: bytes to the next 64-column block
  __device__ __forceinline__ uint64_t desc(int kstep) const {
    if (swizzled)
      return smem_desc(saddr + kstep * (contract_rows ? 2048u : 32u), contract_rows ? block_stride : 16u, 1024u) |
             (static_cast<uint64_t>(2) << 61);
    if (contract_rows) return smem_desc(saddr + kstep * 256u, 128u, rows * 16u);
    return smem_desc(saddr + kstep * 2u * rows * 16u, rows * 16u, 128u);
  }
  // start-address advance per K = 16 step, in 16-byte units
  __device__ __forceinline__ uint32_t advance() const {
    if (swizzled) return contract_rows ? 128u : 2u;
    return contract_rows ? 16u : 2u * rows;
  }
};
// SW tile operand
__device__ __forceinline__ Operand sw_operand(uint32_t saddr, bool contract_rows, uint32_t block_stride = 16) {
  return Operand{saddr, 0u, contract_rows, true, block_stride};
}

// ---- instructions ----------------------------------------------------------
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t e;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(e));
  return e != 0;
}

// D[M x N] (+)= A B^T-style product over KSTEPS K=16 slices.  Called by ALL lanes of one warp
// with warp-uniform arguments; only the `leader` lane (elect_one()) issues.  Keeping the
// descriptor arithmetic warp-uniform lets it live in uniform registers, and with the K loop
// unrolled the slices differ by immediates: measured 27-33 cycles per M = 64 instruction
// against 78 when a single divergent thread builds and issues them (and that cost is per instruction:
// issuing independent accumulators round-robin instead of one product after the other measured the same).  Only the
// start-address field (low 14 bits, 16-byte units) changes from slice to slice.
template <int KSTEPS>
__device__ __forceinline__ void gemm(uint32_t tmem_d, const Operand& a, const Operand& b, uint32_t idesc,
                                     bool accumulate, bool leader) {
  const uint64_t da = a.desc(0), db = b.desc(0);
  const uint32_t adv_a = a.advance(), adv_b = b.advance();
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    if (leader)
      mma_bf16(tmem_d, da + static_cast<uint64_t>(k * adv_a), db + static_cast<uint64_t>(k * adv_b), idesc,
               (accumulate || k > 0) ? 1u : 0u);
  }
}

// Operand advanced by `half` * 4 K steps (64 columns of a K = 128 contraction).  For an SW tile
// contracted over its columns the second half is the next 64-column block (block_stride bytes on).
__device__ __forceinline__ Operand k_half(Operand o, int half) {
  if (o.swizzled && !o.contract_rows) o.saddr += half * o.block_stride;
  else o.saddr += half * 4 * o.advance() * 16;
  return o;
}
// K = 128 contraction as two runs of four K steps, so that SW tiles (two 64-column blocks) and panel
// operands can be mixed.
__device__ __forceinline__ void gemm128(uint32_t tmem_d, const Operand& a, const Operand& b, uint32_t idesc,
                                        bool accumulate, bool leader) {
  gemm<4>(tmem_d, k_half(a, 0), k_half(b, 0), idesc, accumulate, leader);
  gemm<4>(tmem_d, k_half(a, 1), k_half(b, 1), idesc, true, leader);
}

__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Makes generic-proxy shared-memory writes visible to the tensor core (async proxy).
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(columns) : "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Waits for the phase with the given parity.  Each poll lets the hardware suspend
// the thread for up to ~1 ms or until the phase completes (suspend-time hint), so
// waiting threads do not burn issue slots re-polling; after `limit` polls (about a
// second) the wait gives up and returns false -- the caller records it and carries
// on, so a kernel can never spin forever.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = 1024) {
  uint32_t ok = 0;
  for (int it = 0; it < limit && !ok; ++it) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(1000000u)
        : "memory");
  }
  return ok != 0;
}

// The form the kernels use: records a wait that gave up in `timed_out`, and once one has, later
// waits of the same thread poll only once, so a kernel whose copies or MMAs never complete still
// drains in about a second instead of a second per wait.
__device__ __forceinline__ void mbar_wait_flag(uint64_t* bar, uint32_t parity, bool& timed_out) {
  if (!mbar_wait(bar, parity, timed_out ? 1 : 1024)) timed_out = true;
}

// ---- TMEM <-> registers (each thread: its own lane, 8 consecutive columns) ----
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* out) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const float* in) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(__float_as_uint(in[0])), "r"(__float_as_uint(in[1])), "r"(__float_as_uint(in[2])),
               "r"(__float_as_uint(in[3])), "r"(__float_as_uint(in[4])), "r"(__float_as_uint(in[5])),
               "r"(__float_as_uint(in[6])), "r"(__float_as_uint(in[7]))
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Reads N (multiple of 8) consecutive fp32 columns of this thread's TMEM lane.
template <int N>
__device__ __forceinline__ void tmem_ld_row(uint32_t taddr, float* out) {
#pragma unroll
  for (int c = 0; c < N; c += 8) tmem_ld8(taddr + c, out + c);
  tmem_ld_wait();
}

// ---- bf16 packing ----------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint4 pack8_bf16(const float* x) {
  return make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
}
__device__ __forceinline__ void unpack8_bf16(uint4 v, float* x) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

}  // namespace umma
}  // namespace mxk
