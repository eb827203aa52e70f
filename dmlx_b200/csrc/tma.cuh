// Host helper: build TMA tensor maps without linking libcuda (the encoder is fetched from the
// driver at run time), and the device-side tiled-load wrappers.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "common.h"
#include "ptx.cuh"

// rank-`rank` row-major tensor of `elem_bytes`-sized elements; dims/box innermost first;
// strides in bytes for dims 1..rank-1.  128-byte swizzle, zero fill out of bounds.
b200_status b200_make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                                 const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box);

namespace ptx {
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
}  // namespace ptx
