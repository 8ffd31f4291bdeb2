// out[M, N] = X[M, K] * W[N, K]^T for up to eight rows M (decode steps) and a weight with many rows, without
// any sum across thread blocks: a block owns up to 128 rows of W for the whole of K.
//
//   - the grid is one block per multiprocessor where the weight allows it (16 to 128 rows a block); a block
//     has eight computing warps and one that copies: one thread of it issues TMA loads (cp.async.bulk.tensor,
//     128-byte swizzle) of the block's rows, 64 k at a time, into a deep ring of shared-memory stages.  The
//     first ring-full is requested BEFORE the kernel waits for its predecessor on the stream (no kernel
//     writes weights); the activations (all of X, a few KB) follow after the wait;
//   - the computing warps split a stage by k: each reads 16 x 16 pieces of W for all of the block's rows and
//     one 16 x 8 piece of X with ldmatrix and multiplies them with mma.sync.m16n8k16 (rows of W on the M
//     side, tokens on the N side), float32 accumulation, one independent chain per 16 rows; four warps share
//     a stage, the other four take the next one, and a stage is freed by their four arrivals on its "empty"
//     mbarrier.  The eight partial sums meet in shared memory at the end;
//   - plain mode stores the 16 x 8 results.  Gated mode expects the weight of a gated feed-forward with its
//     rows in blocks of sixteen, eight of the gate projection followed by the same eight of the up
//     projection, and stores silu(gate) * up for the eight features: the activation costs no kernel and no
//     trip through memory.  (Both factors are rounded to bfloat16 first, as they are where the product and
//     the activation are separate kernels.)
//
// Every wait on an mbarrier is bounded: a wait that does not finish within the limit sets the error flag
// that the host checks, and the block drains and returns.
#include "tcgen05.cuh"

#include <mutex>
#include <unordered_map>

namespace ms {
namespace wide {

using namespace ms::t5;

constexpr int BK = 64, MAX_TILES = 8, MAX_STAGES = 16, X_ROWS = 8, COMPUTE_WARPS = 8, THREADS = 32 * (COMPUTE_WARPS + 1);
constexpr int SMEM_BUDGET = 180 * 1024;      // of 227 KB: what is left lets the next kernel's blocks start early

enum : int { MODE_PLAIN = 0, MODE_GATED = 1 };

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

template <int MODE, typename OutT>
__global__ void __launch_bounds__(THREADS)
gemm_wide_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 OutT* __restrict__ out, int M, int N, int K, int tiles, int stages, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], x_full;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kc = (K + BK - 1) / BK;
  const int rows = tiles * 16;                     // rows of W per block
  const int stage_bytes = rows * 128;
  unsigned char* x_s = smem;                       // kc chunks of [8 tokens x 64 k]
  unsigned char* ring = smem + (size_t)kc * (X_ROWS * 128);
  const int row0 = blockIdx.x * rows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);                 // the four warps that read a stage
    }
    mbar_init(&x_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dependency_launch();

  if (warp == COMPUTE_WARPS) {
    if (lane == 0) {
      // ---------------- copies
      const int ahead = kc < stages ? kc : stages;
      for (int i = 0; i < ahead; ++i) {            // weights first: nothing on the stream writes them
        mbar_expect_tx(&full_bar[i], stage_bytes);
        tma_load_2d(ring + (size_t)i * stage_bytes, &map_w, &full_bar[i], i * BK, row0);
      }
      grid_dependency_wait();                      // X comes from the kernel before this one
      mbar_expect_tx(&x_full, kc * (X_ROWS * 128));
      for (int i = 0; i < kc; ++i) tma_load_2d(x_s + (size_t)i * (X_ROWS * 128), &map_x, &x_full, i * BK, 0);
      bool ok = true;
      int i = ahead;
      for (; i < kc; ++i) {
        const int stage = i % stages;
        if (!(ok = mbar_wait(&empty_bar[stage], ((i / stages) & 1) ^ 1, error_flag, 1))) break;
        mbar_expect_tx(&full_bar[stage], stage_bytes);
        tma_load_2d(ring + (size_t)stage * stage_bytes, &map_w, &full_bar[stage], i * BK, row0);
      }
      if (!ok || *reinterpret_cast<volatile int*>(error_flag) != 0) {
        // something gave up: let the copies still in flight land before the block may exit
        for (int j = i - 1; j >= 0 && j >= i - stages; --j) mbar_wait(&full_bar[j % stages], (j / stages) & 1, error_flag, 4);
        mbar_wait(&x_full, 0, error_flag, 4);
      }
    }
    // The other lanes of this warp do nothing, and must not wait for the predecessor here: a warp that
    // waits does so as a whole, and lane 0 would be held back from the loads above.
  } else {
    // ---------------- products.  Eight warps: warp w takes the 16 k numbered (w % 4) of every second 64-k
    // stage (w / 4 says which), for all of the block's rows; the eight partial sums meet at the end.
    // A ring that wraps has an even number of stages, so a stage always returns to the same four warps: a
    // warp that waits for a stage's phase by its parity must itself have seen the phase before.
    grid_dependency_wait();
    const int kk = warp & 3, group = warp >> 2;
    float acc[MAX_TILES][4];
#pragma unroll
    for (int t = 0; t < MAX_TILES; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    bool ok = mbar_wait(&x_full, 0, error_flag, 2);
    ok = __all_sync(0xffffffffu, ok);
    const unsigned ring_u32 = smem_u32(ring), x_u32 = smem_u32(x_s);
    const unsigned a_offset = swizzled((lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4));
    const unsigned b_offset = swizzled(lane & 7, 2 * kk + ((lane >> 3) & 1));
    for (int kb = group; kb < kc && ok; kb += 2) {
      const int stage = kb % stages;
      ok = mbar_wait(&full_bar[stage], (kb / stages) & 1, error_flag, 3);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const unsigned w_tile = ring_u32 + (unsigned)(stage * stage_bytes) + a_offset;
      unsigned a[MAX_TILES][4], b[2];
      ldmatrix_x2(b, x_u32 + (unsigned)(kb * (X_ROWS * 128)) + b_offset);
#pragma unroll
      for (int t = 0; t < MAX_TILES; ++t)
        if (t < tiles) ldmatrix_x4(a[t], w_tile + t * 2048);      // sixteen rows further: the swizzle repeats
#pragma unroll
      for (int t = 0; t < MAX_TILES; ++t)
        if (t < tiles) mma_16816(acc[t], a[t], b);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
    // the partial sums go through the ring, which every warp has left by then
    ok = all_compute_warps(ok);
    float4* partial = reinterpret_cast<float4*>(ring);             // [warp][tile][lane]
    if (ok) {
#pragma unroll
      for (int t = 0; t < MAX_TILES; ++t)
        if (t < tiles) partial[(warp * tiles + t) * 32 + lane] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    }
    sync_compute_warps();
    if (ok && warp < tiles) {
      float4 c = partial[warp * 32 + lane];
#pragma unroll
      for (int w = 1; w < COMPUTE_WARPS; ++w) {
        const float4 p = partial[(w * tiles + warp) * 32 + lane];
        c.x += p.x; c.y += p.y; c.z += p.z; c.w += p.w;
      }
      // c.x, c.y: row (lane / 4), tokens 2 (lane % 4) and + 1;  c.z, c.w: the row eight further
      const int r = lane >> 2, t0 = 2 * (lane & 3);
      if (MODE == MODE_GATED) {
        const int feature = (blockIdx.x * tiles + warp) * 8 + r, features = N / 2;
        if (feature < features) {
          if (t0 < M) out[(size_t)t0 * features + feature] = from_float<OutT>(silu_times(round_bf16(c.x), round_bf16(c.z)));
          if (t0 + 1 < M)
            out[(size_t)(t0 + 1) * features + feature] = from_float<OutT>(silu_times(round_bf16(c.y), round_bf16(c.w)));
        }
      } else {
        const int row = row0 + warp * 16 + r;
        if (row < N) {
          if (t0 < M) out[(size_t)t0 * N + row] = from_float<OutT>(c.x);
          if (t0 + 1 < M) out[(size_t)(t0 + 1) * N + row] = from_float<OutT>(c.y);
        }
        if (row + 8 < N) {
          if (t0 < M) out[(size_t)t0 * N + row + 8] = from_float<OutT>(c.z);
          if (t0 + 1 < M) out[(size_t)(t0 + 1) * N + row + 8] = from_float<OutT>(c.w);
        }
      }
    }
  }
}

// Tensor maps are encoded once for each (matrix, shape, box) and kept: a weight keeps its address, and
// the activations come from a few buffers that the caller uses again.
struct MapKey {
  const void* base;
  int rows, K, box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K * 7919u) ^ (size_t)k.box_rows;
  }
};

static bool cached_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> guard(mutex);
  const MapKey key{base, rows, K, box_rows};
  auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

static int multiprocessors() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 1;
  }
  return count;
}

// How the product is laid out: 16-row tiles per block and ring stages; false if it does not fit.
static bool plan(int N, int K, int* tiles, int* stages) {
  const int kc = (K + BK - 1) / BK;
  const long long row_tiles = ((long long)N + 15) / 16;
  long long per_block = (row_tiles + multiprocessors() - 1) / multiprocessors();
  if (per_block > MAX_TILES) per_block = MAX_TILES;      // (more blocks than multiprocessors then)
  if (per_block < 1) per_block = 1;
  const long long x_bytes = (long long)kc * (X_ROWS * 128);
  long long ring = (SMEM_BUDGET - x_bytes) / (per_block * 16 * 128);
  if (ring > MAX_STAGES) ring = MAX_STAGES;
  if (ring >= kc) ring = kc;
  else ring &= ~1LL;     // a stage that is used again must come back to the same half of the computing warps: see the kernel
  if (ring < 4 && ring < kc) return false;
  *tiles = (int)per_block;
  *stages = (int)ring;
  return true;
}

template <int MODE, typename OutT>
int launch(const void* X, const void* W, void* out, int M, int N, int K, int* error_flag, cudaStream_t stream) {
  int tiles = 0, stages = 0;
  MS_REQUIRE(plan(N, K, &tiles, &stages), "gemm_wide: an inner size of %d leaves no room for the weight ring", K);
  CUtensorMap map_w, map_x;
  const bool maps_ok = cached_map(&map_w, W, N, K, tiles * 16) && cached_map(&map_x, X, M, K, X_ROWS);
  MS_REQUIRE(maps_ok, "gemm_wide: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, N, K);
  const int kc = (K + BK - 1) / BK;
  size_t ring = (size_t)stages * tiles * 16 * 128;
  if (ring < (size_t)COMPUTE_WARPS * tiles * 512) ring = (size_t)COMPUTE_WARPS * tiles * 512;     // the partial sums at the end
  const size_t smem = (size_t)kc * (X_ROWS * 128) + ring + 1024;
  auto kernel = gemm_wide_kernel<MODE, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET + 2048);
    if (e != cudaSuccess) MS_FAIL("gemm_wide: cannot reserve shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int blocks = (int)(((long long)N + tiles * 16 - 1) / (tiles * 16));
  cudaError_t e = ms::launch(kernel, dim3(blocks), dim3(THREADS), smem, stream, map_w, map_x, (OutT*)out, M, N, K,
                             tiles, stages, error_flag);
  if (e != cudaSuccess) MS_FAIL("gemm_wide: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace wide
}  // namespace ms

using namespace ms;

// Whether ms_gemm_wide takes a product with this inner size (the activations and a ring of weight stages
// have to fit in shared memory): 0 no; 1 yes, with more blocks than multiprocessors; 2 yes, with at most one
// block per multiprocessor.
MS_EXPORT int ms_gemm_wide_supports(int N, int K) {
  int tiles = 0, stages = 0;
  if (!(K > 0 && K % 8 == 0 && N > 0 && wide::plan(N, K, &tiles, &stages))) return 0;
  return ((long long)N + tiles * 16 - 1) / (tiles * 16) <= wide::multiprocessors() ? 2 : 1;
}

// X [M, K], W [N, K] bfloat16 (K a multiple of 8, both 16-byte aligned), M <= 8.
//   mode 0: out [M, N], bfloat16 (out_dtype 1) or float32 (0);
//   mode 1: W holds a gated feed-forward's gate and up projections in blocks of sixteen rows (eight gate rows,
//           then the up rows of the same eight features; N a multiple of 16); out [M, N / 2] bfloat16 =
//           silu(gate) * up.
// error_flag: one int on the device, zero before the first call; a kernel that gave up waiting writes a
// non-zero code there (1, 4 copies; 2, 3 products), which the caller checks when it synchronises.
MS_EXPORT int ms_gemm_wide(const void* X, const void* W, void* out, int out_dtype, int mode, int M, int N, int K,
                           int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(M <= wide::X_ROWS, "gemm_wide: %d rows; this kernel takes at most %d", M, wide::X_ROWS);
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_wide: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_wide: operands must be 16-byte aligned");
  MS_REQUIRE(error_flag != nullptr, "gemm_wide: an error flag on the device is required");
  if (mode == wide::MODE_GATED) {
    MS_REQUIRE(N % 16 == 0 && out_dtype == MS_BF16, "gemm_wide: gated mode wants a multiple of 16 rows (%d) and bfloat16 results", N);
    return wide::launch<wide::MODE_GATED, __nv_bfloat16>(X, W, out, M, N, K, error_flag, stream);
  }
  MS_REQUIRE(mode == wide::MODE_PLAIN, "gemm_wide: unknown mode %d", mode);
  if (out_dtype == MS_BF16) return wide::launch<wide::MODE_PLAIN, __nv_bfloat16>(X, W, out, M, N, K, error_flag, stream);
  if (out_dtype == MS_F32) return wide::launch<wide::MODE_PLAIN, float>(X, W, out, M, N, K, error_flag, stream);
  MS_FAIL("gemm_wide: unknown output type code %d", out_dtype);
}
