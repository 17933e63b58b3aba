// TMA (cp.async.bulk.tensor) helpers: host-side tensor-map encoding and the device-side tiled load that lands
// a [rows x 64] 16-bit box in shared memory in the 128-byte-swizzled layout tcgen05.mma reads (umma.cuh).
// No multicast is used anywhere: every CTA fetches its own tiles.
#pragma once

#include <cuda.h>

#include "umma.cuh"

namespace jla {
namespace tma {

// ---- host ---------------------------------------------------------------------------------------------------
// Tensor map over a 16-bit tensor seen as [outer][mid][inner] (row-major, `inner` contiguous) with box
// {64 inner elements, 1, box_rows outer rows} and 128-byte swizzle. `mid` = 1 gives a plain 2-D matrix.
// Returns false (and sets the library error text) when the driver entry point is missing or rejects the shape.
bool encode_3d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t mid, uint64_t outer, uint32_t box_rows);

// ---- device -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(umma::smem_addr(bar)), "r"(bytes)
               : "memory");
}

// One box: inner coordinate c_inner (multiple of 8 elements), mid index, outer row. The mbarrier receives the bytes.
__device__ __forceinline__ void load_3d(void* smem_dst, const CUtensorMap* map, int c_inner, int c_mid, int c_outer,
                                        uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::
          "r"(umma::smem_addr(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c_inner), "r"(c_mid), "r"(c_outer), "r"(umma::smem_addr(bar))
      : "memory");
}

// A [ROWS x COLS] tile as COLS / 64 column blocks (the layout of umma::swz_tile); returns the bytes requested.
template <int ROWS, int COLS>
__device__ __forceinline__ uint32_t load_tile(unsigned char* smem_tile, const CUtensorMap* map, int col0, int mid,
                                              int row0, uint64_t* bar) {
#pragma unroll
  for (int cb = 0; cb < COLS / 64; ++cb) load_3d(smem_tile + cb * ROWS * 128, map, col0 + cb * 64, mid, row0, bar);
  return ROWS * COLS * 2;
}

// Untiled bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned) from global to shared memory.
__device__ __forceinline__ void load_bulk(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   umma::smem_addr(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(umma::smem_addr(bar))
               : "memory");
}

// ---- stores (shared -> global) ------------------------------------------------------------------------------
// One box from a 128-byte-swizzled shared-memory tile to global memory through a tensor map made by encode_3d.
// Issued by ONE thread after the writers of the tile have fenced their generic-proxy writes
// (umma::fence_async_smem) and synchronised with it. Completion is tracked per thread in bulk groups:
// store_commit() closes a group, store_wait_read<N>() returns once all but the N newest groups have finished
// READING shared memory (the tile may be overwritten), store_wait<N>() once they are complete in global memory.
// The inner coordinate must be a multiple of 8 elements and no coordinate may be negative.
__device__ __forceinline__ void store_3d(const CUtensorMap* map, const void* smem_src, int c_inner, int c_mid, int c_outer) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];\n" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(umma::smem_addr(smem_src)), "r"(c_inner), "r"(c_mid), "r"(c_outer)
               : "memory");
}
__device__ __forceinline__ void store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

}  // namespace tma
}  // namespace jla
