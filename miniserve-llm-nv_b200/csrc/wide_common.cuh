// What the few-row product that streams weights through a TMA ring into mma.sync is made of (gemm_wide.cu):
// fragment loads from 128-byte-swizzled tiles, the gated activation, barriers of the computing
// warps, cached tensor maps.
#pragma once

#include "tcgen05.cuh"

#include <mutex>
#include <unordered_map>

namespace ms {
namespace wide {

using namespace ms::t5;

constexpr int BK = 64, MAX_TILES = 8, X_ROWS = 8, COMPUTE_WARPS = 16, THREADS = 32 * (COMPUTE_WARPS + 1);

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned (&r)[2], unsigned address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(address));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Byte offset of the 16-byte chunk `chunk` (of eight k) of row `row` in a tile stored as rows of 128 bytes
// with the 128-byte swizzle, the tile starting on a 1024-byte boundary.
__device__ __forceinline__ unsigned swizzled(int row, int chunk) { return (unsigned)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// silu(g) * u as the separate activation kernel computes it for bfloat16 data.
__device__ __forceinline__ float silu_times(float g, float u) {
  const float e = __expf(-fabsf(g));
  const float r = __fdividef(1.0f, 1.0f + e);
  return g * (g >= 0.f ? r : e * r) * u;
}

// Barriers of the computing warps alone (the copying warp takes no part).
__device__ __forceinline__ bool all_compute_warps(bool ok) {
  unsigned all;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.and.pred q, 1, %2, p;\nselp.u32 %0, 1, 0, q;\n}"
               : "=r"(all) : "r"((unsigned)ok), "n"(32 * COMPUTE_WARPS) : "memory");
  return all != 0;
}
__device__ __forceinline__ void sync_compute_warps() { asm volatile("bar.sync 1, %0;" ::"n"(32 * COMPUTE_WARPS) : "memory"); }

// Tensor maps are encoded once for each (matrix, shape, box) and kept: a weight keeps its address, and
// the activations come from a few buffers that the caller uses again.
struct MapKey {
  const void* base;
  int rows, K, box_rows, box_pieces;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows && box_pieces == o.box_pieces;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K * 7919u) ^ (size_t)k.box_rows ^ ((size_t)k.box_pieces << 20);
  }
};

// box_pieces == 0: a map of the matrix [rows, K] with boxes of box_rows x 64 k.  box_pieces > 0 (K a multiple
// of 64 only): the same memory seen as [K / 64 pieces][rows][64 k], boxes of box_pieces x box_rows x 64: one copy
// brings several 64-k pieces of the same rows, laid out in shared memory piece after piece.
inline bool cached_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows, int box_pieces = 0) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> guard(mutex);
  const MapKey key{base, rows, K, box_rows, box_pieces};
  auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  if (box_pieces > 0 && K % BK != 0) return false;
  const bool pieces = box_pieces > 0;
  const cuuint64_t dims[3] = {(cuuint64_t)(pieces ? BK : K), (cuuint64_t)rows, (cuuint64_t)(K / BK)};
  const cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)BK * 2};
  const cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, (cuuint32_t)box_pieces};
  const cuuint32_t elem[3] = {1, 1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, pieces ? 3 : 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

inline int multiprocessors() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 1;
  }
  return count;
}

}  // namespace wide
}  // namespace ms
