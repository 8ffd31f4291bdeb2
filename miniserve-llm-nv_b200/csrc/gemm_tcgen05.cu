// out[M, N] = X[M, K] * W[N, K]^T on the fifth-generation tensor cores (tcgen05), for the many-row
// products of prompt portions.  bfloat16 operands, float32 accumulation in tensor memory.
//
// One thread block computes one 128 x BN tile of the output:
//   warp 0      one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the X and W
//               tiles of each 64-wide k-block into a ring of shared-memory stages and announces them on
//               per-stage "full" mbarriers;
//   warp 1      allocates BN columns of tensor memory; one thread issues tcgen05.mma (M 128, N BN, K 16,
//               four per k-block) reading the stages through shared-memory descriptors, and releases each
//               stage with tcgen05.commit on its "empty" mbarrier; a last commit announces the accumulator;
//   warps 2..5  read the accumulator out of tensor memory (tcgen05.ld, one output row per thread),
//               apply the epilogue and store.
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
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ unsigned tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_n = blockIdx.x, tile_m = blockIdx.y;
  const int num_k = (K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(BN) : "memory");
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
      // ---------------- producer: TMA loads
      for (int kb = 0; kb < num_k; ++kb) {
        const int stage = kb % STAGES;
        const unsigned phase = (kb / STAGES) & 1;
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, error_flag, 1)) break;
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
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issue
      constexpr unsigned idesc = umma_idesc(BM, BN, W_TRANSPOSED);
      bool ok = true;
      for (int kb = 0; kb < num_k && ok; ++kb) {
        const int stage = kb % STAGES;
        const unsigned phase = (kb / STAGES) & 1;
        ok = mbar_wait(&full_bar[stage], phase, error_flag, 2);
        if (!ok) break;
        tmem_fence_after();
        unsigned char* a_s = smem + (size_t)stage * Layout::STAGE_BYTES;
        unsigned char* b_s = a_s + Layout::A_BYTES;
        const uint64_t a_desc = umma_desc(a_s), b_desc = umma_desc(b_s);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing 16 elements (32 bytes) along K inside the 128-byte swizzled row: +2 in 16-byte units
          if (!W_TRANSPOSED) {
            umma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          } else {
            // 16 k-rows of 128 bytes further per step; the blocks of 64 n are BK * 128 bytes apart
            umma_bf16(tmem_base, a_desc + 2 * k, umma_desc_mn_major(b_s + k * (UMMA_K * 128), BK * 128), idesc,
                      (kb | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&empty_bar[stage]);      // the stage is free once these MMAs have read it
      }
      umma_commit(&accum_bar);               // the accumulator is complete once all MMAs have finished
    }
  } else {
    // ---------------- epilogue: warps 2..5 own the tensor-memory lane quarters 2, 3, 0, 1
    const int quarter = warp & 3;
    const int row = tile_m * BM + quarter * 32 + lane;
    if (mbar_wait(&accum_bar, 0, error_flag, 3)) {
      tmem_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        float v[32];
        tmem_load_32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c, v);
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
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
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
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  MS_REQUIRE(grid.y <= 65535, "gemm_tcgen05: %d rows in one launch is too many", M);
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
  const bool narrow = N <= 2048;      // more, smaller tiles when the output is narrow
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
