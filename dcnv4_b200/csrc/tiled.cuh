// Helpers of the spatially tiled DCNv4 kernels (dcnv4_fwd_tiled.cu, dcnv4_bwd_tiled.cu).
//
// A *task* is one (query tile, group): a th x tw patch of output positions of one image and the
// D = 16 channels of one group.  One warp executes a task:
//  * the BH x BW pixel box of `value` that the tile's sampling points can land in (tile + halo)
//    is copied into shared memory by ONE tiled TMA load (cp.async.bulk.tensor.4d over this GPU's
//    own memory, no multicast; out-of-image pixels arrive as zeros, which is exactly the
//    operator's zero padding), group-major, so the two horizontally adjacent corners of a sample
//    are one contiguous span;
//  * a sampling point is handled by a quarter-warp (8 lanes): lanes 0-3 own the four channel
//    quads of the left corner, lanes 4-7 those of the right corner, so that a 128-bit access
//    of a quarter-warp covers one contiguous 128-byte span of fp32 data -- every shared-memory
//    bank exactly once, no conflicts whatever the sampling position;
//  * per-point quantities (corner offset inside the box, bilinear fractions, mask) are computed
//    ONCE, by one lane per point (32 points per pass), and handed to the quarter-warps through
//    a 512-byte record buffer, instead of being recomputed by every lane of a pair;
//  * a point whose footprint leaves the box takes a slower path through global memory.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace dcnb200 {

// Flags in the low six bits of a point record's first word.
constexpr int kRecDead = 1;      // no contribution (query outside the tile, or point failed the range test)
constexpr int kRecOutside = 2;   // footprint leaves the staged box: go through global memory
constexpr int kRecRoundShift = 2;   // bits 2-3: round in which this point runs (collision-free schedule)
constexpr int kRecRoundsShift = 4;  // bits 4-5: rounds of its group of four, minus one

// Largest image side the record packing supports (13 bits for row + 1 and for column + 1).
constexpr int kTiledMaxSide = 8190;

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ float4 lds_f4(const void* base, int byte_off) {
  return *reinterpret_cast<const float4*>(static_cast<const unsigned char*>(base) + byte_off);
}
__device__ __forceinline__ void sts_f4(void* base, int byte_off, float4 v) {
  *reinterpret_cast<float4*>(static_cast<unsigned char*>(base) + byte_off) = v;
}

// Four channels of one corner from the staged box; `fp32_off` is the byte offset the same
// channels have in an fp32 box of the same geometry.
__device__ __forceinline__ float4 lds_val4(const float* box, int fp32_off) { return lds_f4(box, fp32_off); }
__device__ __forceinline__ float4 lds_val4(const __half* box, int fp32_off) {
  const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(box) + (fp32_off >> 1));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 lds_val4(const __nv_bfloat16* box, int fp32_off) {
  const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(box) + (fp32_off >> 1));
  return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u), __uint_as_float(r.y << 16),
                     __uint_as_float(r.y & 0xffff0000u));
}

// Host side: 4-D tensor map over a channels-last (N, H, W, C) tensor with a (1, BH, BW, 16) box.
// Returns false when the driver has no tensor-map support.
bool make_value_map(CUtensorMap* m, int dtype, const void* base, int N, int H, int W, int C, int box_h, int box_w);

// Tile size of the tiled kernels for an output extent: at most `max_tile`, as even as the extent allows.
inline int tiled_tile_extent(int out, int max_tile) {
  const int n = (out + max_tile - 1) / max_tile;
  return (out + n - 1) / n;
}

}  // namespace dcnb200
