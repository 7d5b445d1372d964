// Tensor-memory-accelerator (TMA) plumbing: host-side tensor-map construction
// for [B][T][H][D] bf16 tensors and the device-side issue / completion wrappers.
//
// The "panel" shared-memory format of umma.cuh, [c / 8][t][8], is exactly what a
// tiled TMA load writes when the tensor is described with dimensions ordered
// (8 elements, t, c / 8, h, b): the box {8, rows, D / 8, 1, 1} lands in shared
// memory with the first box dimension fastest, so one instruction issued by one
// thread fetches a whole rows x D tile in tensor-core operand order, zero-filling
// rows past the end of the sequence.  The innermost coordinate is always 0, so the
// 16-byte alignment rule of TMA copies holds by construction.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "umma.cuh"

namespace mxk {
namespace tma {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, looked up through the runtime so that the library does
// not link against the driver; nullptr when it cannot be found.
inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Map whose loads write `rows` x D tiles of one (b, h) sequence in panel order [c/8][t][8].
// Coordinates of a load: {0, t0, 0, h, b}.
inline bool make_panel_map(CUtensorMap* map, const void* base, int B, int T, int H, int D, int rows, int box_panels = 0) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(H) * D * 2;
  const cuuint64_t dims[5] = {8, static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(D / 8), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[4] = {row_bytes, 16, static_cast<cuuint64_t>(D) * 2, row_bytes * T};
  // box_panels (default D / 8) may exceed D / 8: the panels past the tensor are zero-filled
  const cuuint32_t box[5] = {8, static_cast<cuuint32_t>(rows), static_cast<cuuint32_t>(box_panels > 0 ? box_panels : D / 8), 1, 1};
  const cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map whose loads write `rows` x box_cols tiles row-major, [t][box_cols].  Coordinates: {0, h, t0, b}.
// box_cols (default D) may exceed D: the columns past D are zero-filled on loads and clipped on stores,
// which is how a head of 64 columns is served by a kernel built for 128.
inline bool make_plain_map(CUtensorMap* map, const void* base, int B, int T, int H, int D, int rows, int box_cols = 0) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  if (box_cols <= 0) box_cols = D;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(H) * D * 2;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(D) * 2, row_bytes, row_bytes * T};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(box_cols), 1, static_cast<cuuint32_t>(rows), 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map whose loads write `rows` x 64 column blocks of a [B][T][H][D] tensor as 128-byte-swizzled row-major
// lines (umma.cuh "SW tiles"): 128-byte pieces, about five times faster per byte than the panel map.
// Coordinates {c0, h, t0, b} with c0 the first column of the block (a multiple of 64); the destination
// must be 1024-byte aligned.
inline bool make_sw_map(CUtensorMap* map, const void* base, int B, int T, int H, int rows, int D = 64) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(H) * D * 2;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(D) * 2, row_bytes, row_bytes * T};
  const cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(rows), 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef __CUDACC__
// Announces `bytes` of asynchronous copies that will complete on `bar` (one arrival).
__device__ __forceinline__ void expect_bytes(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(umma::smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void load_panel_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int t0, int h, int b) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::
          "r"(umma::smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(umma::smem_u32(bar)), "r"(0), "r"(t0), "r"(0), "r"(h), "r"(b)
      : "memory");
}
__device__ __forceinline__ void load_plain_tile(void* dst, const CUtensorMap* map, uint64_t* bar, int t0, int h, int b,
                                                int c0 = 0) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::
          "r"(umma::smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(umma::smem_u32(bar)), "r"(c0), "r"(h), "r"(t0), "r"(b)
      : "memory");
}
// Contiguous copy; both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void load_bulk(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   umma::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(umma::smem_u32(bar))
               : "memory");
}
// ---- global -> L2 only: the tile a later load_*_tile will fetch, requested a chunk ahead so that the
//      load itself finds it in L2 (no shared memory, no barrier, no completion to wait for).
//      Coordinates follow the alignment rule of the loads (innermost one a multiple of 16 bytes). ----
__device__ __forceinline__ void prefetch_plain_tile(const CUtensorMap* map, int t0, int h, int b, int c0 = 0) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(h), "r"(t0), "r"(b)
               : "memory");
}
__device__ __forceinline__ void prefetch_panel_tile(const CUtensorMap* map, int t0, int h, int b) {
  asm volatile("cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(0), "r"(t0), "r"(0), "r"(h), "r"(b)
               : "memory");
}
// Contiguous range; `src` 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void prefetch_bulk(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// ---- shared -> global (bulk groups of the issuing thread) ----
// Tile store through a plain map; rows past the end of the sequence are clipped.
__device__ __forceinline__ void store_plain_tile(const CUtensorMap* map, const void* src, int t0, int h, int b,
                                                 int c0 = 0) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(umma::smem_u32(src)), "r"(c0), "r"(h), "r"(t0), "r"(b)
               : "memory");
}
__device__ __forceinline__ void store_bulk(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(umma::smem_u32(src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once all but the newest N groups of this thread have finished READING shared memory.
template <int N>
__device__ __forceinline__ void wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Returns once every group of this thread has completed.
__device__ __forceinline__ void wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
#endif

}  // namespace tma
}  // namespace mxk
