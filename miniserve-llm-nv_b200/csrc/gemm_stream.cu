// out[M, N] = X[M, K] * W[N, K]^T for few rows M (decode steps), as a stream of the weight through the
// fifth-generation tensor cores.  bfloat16 operands, float32 accumulation in tensor memory.
//
// Such a product reads every weight once and is bound by memory bandwidth; what a short kernel loses is
// the time before the stream is up to speed.  So:
//   - W is cut into units of 256 rows x 64 k (32 KB).  The grid is one thread block per multiprocessor, and
//     block c takes the units [c U / G, (c + 1) U / G) of the flat list (tile-major), whatever tiles
//     they fall into: every block streams the same number of bytes;
//   - one thread issues the TMA loads into a ring of shared-memory stages that fills nearly all of the
//     shared memory.  The loads of W for the first ring-full are issued BEFORE the kernel waits for its
//     predecessor on the stream (no kernel writes weights), so the stream is already running, or done,
//     when the activations arrive; X follows after the wait;
//   - one thread issues the MMAs.  The 256 weight rows of a unit take the N side of tcgen05.mma and the
//     tokens its M side (M = 64): an MMA has a cost of its own that does not shrink with its size, so the
//     wide side goes to the weights, of which each MMA then consumes 8 KB.  (With the weights on the M
//     side and 16 tokens on the N side the MMAs, not the memory, set the pace: 4 TB/s.)
//   - the accumulator [64 tokens, 256 features] lies in tensor memory, of which a warp reads only its own
//     quarter of the lanes (sixteen tokens for M = 64).  With up to 16 tokens the X tile holds them four
//     times (up to 32: twice), so that every quarter has all tokens and each of the four read-out warps
//     takes a quarter (half) of the features; two accumulators let the next tile start meanwhile.
// A tile whose units are spread over several blocks is summed through a workspace in global memory:
// each block writes its partial sums there and takes a ticket; the block that draws the last ticket adds
// the partial sums in block order, so the result does not depend on timing.  A block has at most two
// such partial tiles, its first and its last.
//
// Every wait on an mbarrier is bounded: a wait that does not finish within the limit sets the error
// flag that the host checks, and the kernel drains and returns (tensor memory is freed on every path).
#include "tcgen05.cuh"

#include <mutex>
#include <unordered_map>

namespace ms {
namespace wstream {

using namespace ms::t5;

constexpr int BN = 256, BK = 64, MT = 64, UMMA_K = 16;
constexpr int THREADS = 192;                 // warp 0 loads, warp 1 issues MMAs, warps 2..5 read out
constexpr int ACC_BUFS = 2;
constexpr int W_BYTES = BN * BK * 2, X_BYTES = MT * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int STAGES = 5;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024;   // + room to align to 1024 bytes

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// First unit of block c, and the block that holds unit u, of U units spread over G blocks.
__device__ __forceinline__ long long first_unit(long long c, long long U, long long G) { return c * U / G; }
__device__ __forceinline__ int block_of_unit(long long u, long long U, long long G) { return (int)(((u + 1) * G + U - 1) / U - 1); }

// Thirty-two consecutive features of one token to `dst`, of which `valid` exist.
template <typename OutT>
__device__ __forceinline__ void store_32(OutT* dst, const float (&v)[32], int valid, bool vector_ok) {
  if (valid >= 32 && vector_ok) {
    if (sizeof(OutT) == 2) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 packed;
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) pairs[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
        *reinterpret_cast<uint4*>(dst + i) = packed;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = from_float<OutT>(v[i]);
  }
}

template <int NT, typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   OutT* __restrict__ out, int M, int N, int K, float* __restrict__ workspace,
                   int* __restrict__ tickets, int* __restrict__ error_flag) {
  constexpr int COPIES = MT / NT;                  // how often the X tile holds the tokens
  constexpr int WARPS_PER_COPY = NT / 16;          // read-out warps that share one copy (sixteen tokens each)
  constexpr int COLS_PER_WARP = BN / COPIES;       // features a read-out warp takes
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[ACC_BUFS], acc_empty[ACC_BUFS];
  __shared__ unsigned tmem_base_s;
  __shared__ int last_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kc = (K + BK - 1) / BK;
  const long long U = (long long)((N + BN - 1) / BN) * kc, G = gridDim.x;
  const long long u0 = first_unit(blockIdx.x, U, G), u1 = first_unit(blockIdx.x + 1, U, G);
  const int n_units = (int)(u1 - u0);

  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);         // one arrival per read-out warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ACC_BUFS * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const unsigned tmem_base = tmem_base_s;
  grid_dependency_launch();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer
      const int ahead = n_units < STAGES ? n_units : STAGES;
      for (int i = 0; i < ahead; ++i) {          // weights first: nothing on the stream writes them
        const long long u = u0 + i;
        mbar_expect_tx(&full_bar[i], STAGE_BYTES);
        tma_load_2d(smem + (size_t)i * STAGE_BYTES, &map_w, &full_bar[i], (int)(u % kc) * BK, (int)(u / kc) * BN);
      }
      grid_dependency_wait();                    // X comes from the kernel before this one
      for (int i = 0; i < ahead; ++i)
#pragma unroll
        for (int c = 0; c < COPIES; ++c)
          tma_load_2d(smem + (size_t)i * STAGE_BYTES + W_BYTES + c * (NT * BK * 2), &map_x, &full_bar[i],
                      (int)((u0 + i) % kc) * BK, 0);
      bool ok = true;
      int i = ahead;
      for (; i < n_units; ++i) {
        const int stage = i % STAGES;
        if (!(ok = mbar_wait(&empty_bar[stage], ((i / STAGES) & 1) ^ 1, error_flag, 1))) break;
        const long long u = u0 + i;
        unsigned char* w_s = smem + (size_t)stage * STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
        tma_load_2d(w_s, &map_w, &full_bar[stage], (int)(u % kc) * BK, (int)(u / kc) * BN);
#pragma unroll
        for (int c = 0; c < COPIES; ++c)
          tma_load_2d(w_s + W_BYTES + c * (NT * BK * 2), &map_x, &full_bar[stage], (int)(u % kc) * BK, 0);
      }
      if (!ok || *reinterpret_cast<volatile int*>(error_flag) != 0) {
        // something gave up: let the copies still in flight land before the block may exit
        for (int j = i - 1; j >= 0 && j >= i - STAGES; --j) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1, error_flag, 4);
      }
    }
    // The other lanes of this warp do nothing, and must not wait for the predecessor here: a warp that
    // waits does so as a whole, and lane 0 would be held back from the loads above.
  } else if (warp == 1) {
    grid_dependency_wait();
    if (lane == 0) {
      // ---------------- MMA issue
      constexpr unsigned idesc = umma_idesc(MT, BN);
      int segment = 0;
      for (int i = 0; i < n_units; ++i) {
        const int kchunk = (int)((u0 + i) % kc);
        const bool first = i == 0 || kchunk == 0, last = i == n_units - 1 || kchunk == kc - 1;
        const int buf = segment % ACC_BUFS;
        if (first && !mbar_wait(&acc_empty[buf], ((segment / ACC_BUFS) & 1) ^ 1, error_flag, 5)) break;
        const int stage = i % STAGES;
        if (!mbar_wait(&full_bar[stage], (i / STAGES) & 1, error_flag, 2)) break;
        tmem_fence_after();
        unsigned char* w_s = smem + (size_t)stage * STAGE_BYTES;
        const uint64_t a_desc = umma_desc(w_s + W_BYTES), b_desc = umma_desc(w_s);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_base + buf * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (first && k == 0) ? 0u : 1u);
        umma_commit(&empty_bar[stage]);
        if (last) {
          umma_commit(&acc_full[buf]);
          ++segment;
        }
      }
    }
  } else {
    // ---------------- read-out: warps 2..5 own the tensor-memory lane quarters 2, 3, 0, 1; with M = 64 a
    // quarter holds sixteen rows of the accumulator in its first sixteen lanes
    grid_dependency_wait();
    const int quarter = warp & 3;
    const int token = 16 * (quarter % WARPS_PER_COPY) + lane;
    const int col0 = (quarter / WARPS_PER_COPY) * COLS_PER_WARP;
    const bool mine_valid = lane < 16 && token < M;
    const int tid = threadIdx.x - 64;              // 0..127 among the read-out threads
    const bool leader = tid == 0;
    const bool out_vector_ok = (N * sizeof(OutT)) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    bool ok = true;
    int segment = 0;
    for (long long u = u0; u < u1; ++segment) {
      const int tile = (int)(u / kc);
      const long long tile_begin = (long long)tile * kc, tile_end = tile_begin + kc;
      const long long end = u1 < tile_end ? u1 : tile_end;
      const bool whole = u == tile_begin && end == tile_end;
      const int buf = segment % ACC_BUFS;
      const int me = blockIdx.x;
      float* mine = workspace + ((size_t)(me * 2 + (segment == 0 ? 0 : 1)) * NT) * BN;
      ok = ok && mbar_wait(&acc_full[buf], (segment / ACC_BUFS) & 1, error_flag, 3);
      ok = __all_sync(0xffffffffu, ok);            // the loads below want the whole warp
      if (ok) {
        tmem_fence_after();
#pragma unroll 1
        for (int c = 0; c < COLS_PER_WARP; c += 32) {
          float v[32];
          tmem_load_32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN + col0 + c), v);
          if (mine_valid) {
            const int col = tile * BN + col0 + c;              // first of these 32 features
            if (whole) {
              if (col < N) store_32<OutT>(out + (size_t)token * N + col, v, N - col, out_vector_ok);
            } else {
              store_32<float>(mine + token * BN + col0 + c, v, 32, true);
            }
          }
        }
        tmem_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      }
      if (!whole) {
        // the barriers below are passed by all four warps whatever happened, so that none waits alone
        __threadfence();
        epilogue_barrier();
        const int first_block = block_of_unit(tile_begin, U, G), last_block = block_of_unit(tile_end - 1, U, G);
        if (leader) {
          const int ticket = atomicAdd(&tickets[tile], 1);
          const int is_last = ticket == last_block - first_block;
          if (is_last) tickets[tile] = 0;         // every other block has drawn: ready for the next launch
          last_s = is_last;
        }
        epilogue_barrier();
        if (last_s && ok) {
          __threadfence();
          // every block but the first of the tile starts inside it (its partial sums are its first ones)
          const int first_which = first_unit(first_block, U, G) >= tile_begin ? 0 : 1;
          // the M x 256 sums as float4 groups, spread over the 128 threads
          for (int g = tid; g < M * (BN / 4); g += 128) {
            const int tok = g / (BN / 4), col = (g % (BN / 4)) * 4;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int b0 = first_block; b0 <= last_block; b0 += 4) {
              float4 part[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {        // the loads of four blocks are in flight before any is added
                const int b = b0 + j;
                const float* theirs = workspace + ((size_t)(b * 2 + (b == first_block ? first_which : 0)) * NT) * BN;
                part[j] = b <= last_block ? __ldcg(reinterpret_cast<const float4*>(theirs + tok * BN + col))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                sum.x += part[j].x; sum.y += part[j].y; sum.z += part[j].z; sum.w += part[j].w;
              }
            }
            const int n = tile * BN + col;
            OutT* dst = out + (size_t)tok * N + n;
            if (n + 4 <= N && N % 4 == 0 && out_vector_ok) {
              if (sizeof(OutT) == 2) {
                uint2 packed;
                __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
                pairs[0] = __floats2bfloat162_rn(sum.x, sum.y);
                pairs[1] = __floats2bfloat162_rn(sum.z, sum.w);
                *reinterpret_cast<uint2*>(dst) = packed;
              } else {
                *reinterpret_cast<float4*>(dst) = sum;
              }
            } else {
              const float s[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (n + i < N) dst[i] = from_float<OutT>(s[i]);
            }
          }
        }
        epilogue_barrier();                        // last_s is free for the next partial tile
      }
      u = end;
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACC_BUFS * BN) : "memory");
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

// A [rows, K] bfloat16 row-major matrix seen by TMA as boxes of 64 k x box_rows rows, 128-byte swizzled;
// what lies outside the matrix reads as zero.
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

template <int NT, typename OutT>
int launch(const void* X, const void* W, void* out, int M, int N, int K, float* workspace, int* tickets,
           int* error_flag, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  const bool maps_ok = cached_map(&map_w, W, N, K, BN) && cached_map(&map_x, X, M, K, NT);
  MS_REQUIRE(maps_ok, "gemm_stream: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, N, K);
  auto kernel = gemm_stream_kernel<NT, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) MS_FAIL("gemm_stream: cannot reserve %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  const long long units = (long long)((N + BN - 1) / BN) * ((K + BK - 1) / BK);
  const int blocks = (int)(units < multiprocessors() ? units : multiprocessors());
  cudaError_t e = ms::launch(kernel, dim3(blocks), dim3(THREADS), SMEM_BYTES, stream, map_w, map_x, (OutT*)out, M, N, K,
                             workspace, tickets, error_flag);
  if (e != cudaSuccess) MS_FAIL("gemm_stream: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace wstream
}  // namespace ms

using namespace ms;

// Most rows of X the streaming product takes.
MS_EXPORT int ms_gemm_stream_max_rows() { return wstream::MT; }

// Sizes of the buffers a caller keeps for the streaming product on one device: `workspace_floats` float32
// values (contents arbitrary) and `ticket_ints` int32 values (zero before the first call; the kernel leaves
// them zero) for a weight of up to `max_weight_rows` rows.
MS_EXPORT int ms_gemm_stream_buffers(int max_weight_rows, long long* workspace_floats, long long* ticket_ints) {
  *workspace_floats = (long long)wstream::multiprocessors() * 2 * wstream::MT * wstream::BN;
  *ticket_ints = (max_weight_rows + wstream::BN - 1) / wstream::BN;
  return 0;
}

// X [M, K], W [N, K] bfloat16 (K a multiple of 8, both 16-byte aligned), M <= 64; out [M, N] bfloat16
// (out_dtype 1) or float32 (out_dtype 0).  `workspace` and `tickets` as ms_gemm_stream_buffers() sizes
// them, with at least ceil(N / 256) tickets; calls that share them must be on one stream.
// error_flag: one int on the device, zero before the first call; a kernel that gave up waiting writes a
// non-zero code there (1 loads, 2 and 5 MMA issue, 3 read-out, 4 draining), which the caller checks when
// it synchronises.
MS_EXPORT int ms_gemm_stream(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K,
                             float* workspace, int* tickets, int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(M <= wstream::MT, "gemm_stream: %d rows; this kernel takes at most %d", M, wstream::MT);
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_stream: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_stream: operands must be 16-byte aligned");
  MS_REQUIRE(workspace != nullptr && tickets != nullptr && error_flag != nullptr,
             "gemm_stream: workspace, tickets and an error flag on the device are required");
  MS_REQUIRE(out_dtype == MS_BF16 || out_dtype == MS_F32, "gemm_stream: unknown output type code %d", out_dtype);
#define MS_STREAM_CASE(NT)                                                                                       \
  return out_dtype == MS_BF16                                                                                    \
             ? wstream::launch<NT, __nv_bfloat16>(X, W, out, M, N, K, workspace, tickets, error_flag, stream)     \
             : wstream::launch<NT, float>(X, W, out, M, N, K, workspace, tickets, error_flag, stream)
  if (M <= 16) { MS_STREAM_CASE(16); }
  if (M <= 32) { MS_STREAM_CASE(32); }
  MS_STREAM_CASE(64);
#undef MS_STREAM_CASE
}
