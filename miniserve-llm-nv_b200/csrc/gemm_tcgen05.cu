// out[M, N] = X[M, K] * W[N, K]^T on the fifth-generation tensor cores (tcgen05), for the many-row
// products of prompt portions.  bfloat16 operands, float32 accumulation in tensor memory.
//
// One thread block per multiprocessor walks over 128 x BN tiles of the output (tile blockIdx.x, then every
// gridDim.x-th; tiles that are neighbours in this order share their W tile, so the blocks running at a time
// read few different W tiles):
//   warp 0      one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the X and W
//               tiles of each 64-wide k-block into a ring of shared-memory stages and announces them on
//               per-stage "full" mbarriers; it runs on into the next tile while the last is finished;
//   warp 1      allocates tensor memory for two accumulators; one thread issues tcgen05.mma (M 128, N BN,
//               K 16, four per k-block) reading the stages through shared-memory descriptors, and releases
//               each stage with tcgen05.commit on its "empty" mbarrier; a last commit per tile announces
//               the accumulator, and the next tile goes to the other one;
//   warps 2..5  read an accumulator out of tensor memory (tcgen05.ld, one output row per thread),
//               apply the epilogue and store, while the next tile is being accumulated.
// Epilogues: plain store (bfloat16 or float32), or add into a float32 matrix in place (the residual
// stream), which spares a separate pass over it.
//
// Every wait on an mbarrier is bounded: a wait that does not finish within the limit sets the error
// flag that the host checks, and the kernel drains and returns (tensor memory is freed on every path).
#include "tcgen05.cuh"

namespace ms {
namespace t5 {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int THREADS = 192;                 // warps 0..5

enum : int { EPI_STORE = 0, EPI_ADD_F32 = 1 };

template <int BN, int STAGES>
struct SharedLayout {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr size_t TOTAL = (size_t)STAGES * STAGE_BYTES + 1024;   // + room to align to 1024 bytes
};

template <int BN, int STAGES, int EPILOGUE, typename OutT, bool W_TRANSPOSED>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    OutT* __restrict__ out, int M, int N, int K, int* __restrict__ error_flag) {
  using Layout = SharedLayout<BN, STAGES>;
  constexpr int ACCUMULATORS = 2;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[ACCUMULATORS], acc_empty[ACCUMULATORS];
  __shared__ unsigned tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int num_k = (K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < ACCUMULATORS; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);         // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ACCUMULATORS * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const unsigned tmem_base = tmem_base_s;

  grid_dependency_wait();          // X (and, for the adding epilogue, out) come from earlier kernels
  grid_dependency_launch();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer: TMA loads, one running count of k-blocks over all tiles of this block
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int stage = it % STAGES;
          const unsigned phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, error_flag, 1))) break;
          unsigned char* a_s = smem + (size_t)stage * Layout::STAGE_BYTES;
          unsigned char* b_s = a_s + Layout::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Layout::STAGE_BYTES);
          tma_load_2d(a_s, &map_x, &full_bar[stage], kb * BK, tile_m * BM);
          if (!W_TRANSPOSED) {
            tma_load_2d(b_s, &map_w, &full_bar[stage], kb * BK, tile_n * BN);
          } else {
            // W stored [K, N]: one box of 64 n x 64 k per block of 64 output columns
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_s + j * (BK * 128), &map_w, &full_bar[stage], tile_n * BN + j * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issue
      constexpr unsigned idesc = umma_idesc(BM, BN, W_TRANSPOSED);
      int it = 0, done = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++done) {
        const int buf = done % ACCUMULATORS;
        if (!(ok = mbar_wait(&acc_empty[buf], ((done / ACCUMULATORS) & 1) ^ 1, error_flag, 4))) break;
        const unsigned accumulator = tmem_base + buf * BN;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int stage = it % STAGES;
          const unsigned phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&full_bar[stage], phase, error_flag, 2))) break;
          tmem_fence_after();
          unsigned char* a_s = smem + (size_t)stage * Layout::STAGE_BYTES;
          unsigned char* b_s = a_s + Layout::A_BYTES;
          const uint64_t a_desc = umma_desc(a_s), b_desc = umma_desc(b_s);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 elements (32 bytes) along K inside the 128-byte swizzled row: +2 in 16-byte units
            if (!W_TRANSPOSED) {
              umma_bf16(accumulator, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            } else {
              // 16 k-rows of 128 bytes further per step; the blocks of 64 n are BK * 128 bytes apart
              umma_bf16(accumulator, a_desc + 2 * k, umma_desc_mn_major(b_s + k * (UMMA_K * 128), BK * 128), idesc,
                        (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[stage]);      // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);   // the accumulator is complete once all MMAs have finished
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 own the tensor-memory lane quarters 2, 3, 0, 1
    const int quarter = warp & 3;
    int done = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++done) {
      const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
      const int buf = done % ACCUMULATORS;
      const int row = tile_m * BM + quarter * 32 + lane;
      ok = ok && mbar_wait(&acc_full[buf], (done / ACCUMULATORS) & 1, error_flag, 3);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tmem_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float v[32];
        tmem_load_32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN + c), v);
        const int col = tile_n * BN + c;
        if (row < M && col < N) {
          OutT* dst = out + (size_t)row * N + col;
          const bool whole = col + 32 <= N && (N % 8 == 0);
          if (EPILOGUE == EPI_ADD_F32) {
            float* d = reinterpret_cast<float*>(dst);
            if (whole) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 old = *reinterpret_cast<float4*>(d + i);
                old.x += v[i]; old.y += v[i + 1]; old.z += v[i + 2]; old.w += v[i + 3];
                *reinterpret_cast<float4*>(d + i) = old;
              }
            } else {
              for (int i = 0; i < 32 && col + i < N; ++i) d[i] += v[i];
            }
          } else if (sizeof(OutT) == 2) {
            if (whole) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 packed;
                __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int j = 0; j < 4; ++j) pairs[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(dst + i) = packed;
              }
            } else {
              for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = from_float<OutT>(v[i]);
            }
          } else {
            if (whole) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
              for (int i = 0; i < 32 && col + i < N; ++i) dst[i] = from_float<OutT>(v[i]);
            }
          }
        }
      }
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);      // the accumulator may be overwritten
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACCUMULATORS * BN) : "memory");
  }
}

// A [rows, K] bfloat16 row-major matrix seen by TMA as boxes of 64 k x box_rows rows, 128-byte swizzled.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, int EPILOGUE, typename OutT, bool W_TRANSPOSED = false>
int launch(const void* X, const void* W, void* out, int M, int N, int K, int* error_flag, cudaStream_t stream) {
  CUtensorMap map_x, map_w;
  // W as [N, K]: boxes of 64 k x BN rows.  W as [K, N]: a [K rows, N inner] matrix in boxes of 64 n x 64 k.
  const bool maps_ok = make_map(&map_x, X, M, K, BM) &&
                       (W_TRANSPOSED ? make_map(&map_w, W, K, N, BK) : make_map(&map_w, W, N, K, BN));
  MS_REQUIRE(maps_ok, "gemm_tcgen05: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, N, K);
  auto kernel = gemm_tcgen05_kernel<BN, STAGES, EPILOGUE, OutT, W_TRANSPOSED>;
  const size_t smem = SharedLayout<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 1;
  }
  const long long tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  MS_REQUIRE(tiles <= 2147483647LL, "gemm_tcgen05: %lld tiles in one launch is too many", tiles);
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  cudaError_t e = ms::launch(kernel, grid, dim3(THREADS), smem, stream, map_x, map_w, (OutT*)out, M, N, K, error_flag);
  if (e != cudaSuccess) MS_FAIL("gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace t5
}  // namespace ms

using namespace ms;

// X [M, K], W [N, K] bfloat16 (K a multiple of 8, both 16-byte aligned); out [M, N]:
//   epilogue 0: stored as bfloat16 (out_dtype 1) or float32 (out_dtype 0);
//   epilogue 1: added in place into a float32 matrix.
// error_flag: one int on the device, zero before the first call; a kernel that gave up waiting writes a
// non-zero code there (1 producer, 2 MMA issue, 3 epilogue), which the caller checks when it synchronises.
MS_EXPORT int ms_gemm_tcgen05(const void* X, const void* W, void* out, int out_dtype, int epilogue, int M, int N, int K,
                              int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_tcgen05: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tcgen05: operands must be 16-byte aligned");
  MS_REQUIRE(error_flag != nullptr, "gemm_tcgen05: an error flag on the device is required");
  // 128 x 256 tiles unless the narrower 128 x 128 ones fill the multiprocessors' waves better
  int sms = 148;
  {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 148;
  }
  const long long rows = (M + 127) / 128;
  const long long waves_wide = (rows * ((N + 255) / 256) + sms - 1) / sms, waves_narrow = (rows * ((N + 127) / 128) + sms - 1) / sms;
  const bool narrow = waves_narrow * 128 * 5 < waves_wide * 256 * 4;     // (a narrow tile does less per byte it loads)
  if (epilogue == t5::EPI_ADD_F32) {
    MS_REQUIRE(out_dtype == MS_F32, "gemm_tcgen05: the adding epilogue works on a float32 matrix");
    return narrow ? t5::launch<128, 6, t5::EPI_ADD_F32, float>(X, W, out, M, N, K, error_flag, stream)
                  : t5::launch<256, 4, t5::EPI_ADD_F32, float>(X, W, out, M, N, K, error_flag, stream);
  }
  MS_REQUIRE(epilogue == t5::EPI_STORE, "gemm_tcgen05: unknown epilogue %d", epilogue);
  if (out_dtype == MS_BF16)
    return narrow ? t5::launch<128, 6, t5::EPI_STORE, __nv_bfloat16>(X, W, out, M, N, K, error_flag, stream)
                  : t5::launch<256, 4, t5::EPI_STORE, __nv_bfloat16>(X, W, out, M, N, K, error_flag, stream);
  if (out_dtype == MS_F32)
    return narrow ? t5::launch<128, 6, t5::EPI_STORE, float>(X, W, out, M, N, K, error_flag, stream)
                  : t5::launch<256, 4, t5::EPI_STORE, float>(X, W, out, M, N, K, error_flag, stream);
  MS_FAIL("gemm_tcgen05: unknown output type code %d", out_dtype);
}

// The same product with the weight stored input-major: Wt [K, N] bfloat16 (N a multiple of 8), out [M, N]
// bfloat16.  The weight tile is then an MN-major operand of the MMA.
MS_EXPORT int ms_gemm_tcgen05_wt(const void* X, const void* Wt, void* out, int M, int N, int K, int* error_flag,
                                 cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(K > 0 && K % 8 == 0 && N % 8 == 0, "gemm_tcgen05_wt: sizes K %d and N %d must be multiples of 8", K, N);
  MS_REQUIRE(error_flag != nullptr, "gemm_tcgen05_wt: an error flag on the device is required");
  return t5::launch<128, 6, t5::EPI_STORE, __nv_bfloat16, true>(X, Wt, out, M, N, K, error_flag, stream);
}
