// out[M, N] = X[M, K] * W[N, K]^T for few rows M (decode steps: M = requests in the batch <= 64).
//
// Such a product reads every weight once and is bound by memory bandwidth, so the kernel is shaped
// for streaming W: the weight rows take the M side of mma.m16n8k16 (16 rows per thread block), the
// batch the N side (8 columns per tile), and each thread fetches its fragments of W straight from
// global memory with 16-byte loads that bypass L1, several in flight.  A 16-byte load holds eight
// consecutive k of one row; the two MMAs that consume it treat them as the k-slots the fragment
// layout assigns to that thread, and X is loaded with the same assignment, so the products pair up
// the same k (the order of k inside a dot product is a permutation, which a sum does not mind).
// The block's warps split K between them, and for matrices with few rows of W a cluster of up to
// four blocks splits K further; partial sums are added in warp order through shared memory and then in
// block order through the cluster's distributed shared memory, so the result does not depend on
// timing.  float32 accumulation, one rounding at the store.
//
// MODE_SILU_MUL reads X as silu(G[m, k]) * G[m, K + k] from a [M, 2K] matrix (rounded to bfloat16
// first, as the separate activation kernel does), which spares that kernel and its round trip.
#include "common.cuh"

#include <cooperative_groups.h>

namespace ms {

constexpr int SK_WARPS = 8;
enum : int { MODE_PLAIN = 0, MODE_SILU_MUL = 1 };

__device__ __forceinline__ uint4 load_stream_16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// silu(g) * u for two bfloat16 pairs, with the fast exponential and division (the result is rounded to
// bfloat16 anyway), by the same formula as the separate activation kernel.
__device__ __forceinline__ float silu_times_fast(float g, float u) {
  const float e = __expf(-fabsf(g));
  const float r = __fdividef(1.0f, 1.0f + e);
  return g * (g >= 0.f ? r : e * r) * u;
}

__device__ __forceinline__ unsigned silu_mul_pair(unsigned gate, unsigned up) {
  const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gate));
  const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&up));
  const __nv_bfloat162 r = __floats2bfloat162_rn(silu_times_fast(g.x, u.x), silu_times_fast(g.y, u.y));
  return *reinterpret_cast<const unsigned*>(&r);
}

template <int NT, int MODE>
__device__ __forceinline__ void load_x(uint4 (&xb)[NT], const __nv_bfloat16* __restrict__ X, int ldx, int M, int K,
                                       int k, int quad_row, bool k_ok) {
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int m = 8 * j + quad_row;
    xb[j] = make_uint4(0u, 0u, 0u, 0u);
    if (k_ok && m < M) {
      const __nv_bfloat16* row = X + (size_t)m * ldx + k;
      if (MODE == MODE_PLAIN) {
        xb[j] = *reinterpret_cast<const uint4*>(row);
      } else {
        const uint4 g = *reinterpret_cast<const uint4*>(row);
        const uint4 u = *reinterpret_cast<const uint4*>(row + K);
        xb[j] = make_uint4(silu_mul_pair(g.x, u.x), silu_mul_pair(g.y, u.y), silu_mul_pair(g.z, u.z),
                           silu_mul_pair(g.w, u.w));
      }
    }
  }
}

template <int NT, int MODE, typename OutT, bool CLUSTER>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, int ldx, const __nv_bfloat16* __restrict__ W,
                   OutT* __restrict__ out, int M, int N, int K) {
  __shared__ float partial[SK_WARPS][16][8 * NT + 1];
  __shared__ float block_sum_s[CLUSTER ? 16 * 8 * NT : 1];
  namespace cg = cooperative_groups;
  const int k_blocks = CLUSTER ? gridDim.y : 1, k_block = CLUSTER ? blockIdx.y : 0;  // the cluster spans y
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad_row = lane >> 2, quad_col = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int units = (K + 31) / 32;                       // steps of 32 k
  const int parts = SK_WARPS * k_blocks;
  const int per_warp = (units + parts - 1) / parts;
  const int k_begin = min(K, (k_block * SK_WARPS + warp) * per_warp * 32);
  const int k_end = min(K, k_begin + per_warp * 32);

  const bool row_a_ok = n0 + quad_row < N, row_b_ok = n0 + quad_row + 8 < N;
  const __nv_bfloat16* w_a = W + (size_t)(row_a_ok ? n0 + quad_row : 0) * K;
  const __nv_bfloat16* w_b = W + (size_t)(row_b_ok ? n0 + quad_row + 8 : 0) * K;

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  // Two batches of weight fragments are in flight: while one is consumed the next is on its way.  The
  // first batch is requested before the kernel waits for its predecessor: weights depend on no kernel.
  constexpr int UNROLL = 4;
  uint4 wa[UNROLL], wb[UNROLL], next_a[UNROLL], next_b[UNROLL];
  auto fetch = [&](int k0, uint4 (&fa)[UNROLL], uint4 (&fb)[UNROLL]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + 32 * u + 8 * quad_col;
      const bool ok = k + 8 <= k_end;
      fa[u] = (ok && row_a_ok) ? load_stream_16(w_a + k) : make_uint4(0u, 0u, 0u, 0u);
      fb[u] = (ok && row_b_ok) ? load_stream_16(w_b + k) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch(k_begin, wa, wb);
  grid_dependency_wait();
  grid_dependency_launch();
  for (int k0 = k_begin; k0 < k_end; k0 += 32 * UNROLL) {
    fetch(k0 + 32 * UNROLL, next_a, next_b);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = k0 + 32 * u + 8 * quad_col;
      uint4 xb[NT];
      load_x<NT, MODE>(xb, X, ldx, M, K, k, quad_row, k + 8 <= k_end);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        mma_bf16_16816(acc[j], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xb[j].x, xb[j].y);
        mma_bf16_16816(acc[j], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xb[j].z, xb[j].w);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      wa[u] = next_a[u];
      wb[u] = next_b[u];
    }
  }

#pragma unroll
  for (int j = 0; j < NT; ++j) {
    partial[warp][quad_row][8 * j + 2 * quad_col] = acc[j][0];
    partial[warp][quad_row][8 * j + 2 * quad_col + 1] = acc[j][1];
    partial[warp][quad_row + 8][8 * j + 2 * quad_col] = acc[j][2];
    partial[warp][quad_row + 8][8 * j + 2 * quad_col + 1] = acc[j][3];
  }
  __syncthreads();
  if constexpr (!CLUSTER) {                              // no cluster: the block's sum is the result
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += blockDim.x) {
      const int m = i / 16, row = i % 16;
      if (m < M && n0 + row < N) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) sum += partial[w][row][m];
        out[(size_t)m * N + n0 + row] = from_float<OutT>(sum);
      }
    }
  } else {
  for (int i = threadIdx.x; i < 16 * 8 * NT; i += blockDim.x) {
    const int m = i / 16, row = i % 16;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) sum += partial[w][row][m];
    block_sum_s[i] = sum;
  }
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();                      // every block's sums are in its shared memory
  if (k_block == 0) {
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += blockDim.x) {
      const int m = i / 16, row = i % 16;
      if (m < M && n0 + row < N) {
        float sum = block_sum_s[i];
        for (int b = 1; b < k_blocks; ++b) sum += cluster.map_shared_rank(block_sum_s, b)[i];
        out[(size_t)m * N + n0 + row] = from_float<OutT>(sum);
      }
    }
  }
  cluster.sync();                                        // nobody leaves while its sums are being read
  }
}

template <int NT, int MODE, typename OutT>
int launch_skinny_nt(const __nv_bfloat16* x, int ldx, const __nv_bfloat16* w, OutT* o, int M, int N, int K,
                     cudaStream_t stream) {
  const int blocks = (N + 15) / 16;
  // Few rows of W give few blocks: split K over a cluster until about two blocks per SM are in flight,
  // as long as every warp keeps at least 128 k.
  int k_blocks = 1;
  while (k_blocks < 4 && blocks * k_blocks < 2 * 148 && K / (SK_WARPS * k_blocks * 2) >= 128) k_blocks *= 2;
  if (k_blocks == 1) {
    ms::launch(gemm_skinny_kernel<NT, MODE, OutT, false>, blocks, SK_WARPS * 32, 0, stream, x, ldx, w, o, M, N, K);
    MS_CHECK_LAUNCH("gemm_skinny");
    return 0;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(blocks, k_blocks, 1);
  config.blockDim = dim3(SK_WARPS * 32, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 1;
  attribute[0].val.clusterDim.y = k_blocks;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // as ms::launch gives every kernel
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, gemm_skinny_kernel<NT, MODE, OutT, true>, x, ldx, w, o, M, N, K);
  if (e != cudaSuccess) MS_FAIL("gemm_skinny: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

template <int MODE, typename OutT>
int launch_skinny(const void* X, int ldx, const void* W, void* out, int M, int N, int K, cudaStream_t stream) {
  auto x = (const __nv_bfloat16*)X;
  auto w = (const __nv_bfloat16*)W;
  auto o = (OutT*)out;
  if (M <= 8) return launch_skinny_nt<1, MODE, OutT>(x, ldx, w, o, M, N, K, stream);
  if (M <= 16) return launch_skinny_nt<2, MODE, OutT>(x, ldx, w, o, M, N, K, stream);
  if (M <= 32) return launch_skinny_nt<4, MODE, OutT>(x, ldx, w, o, M, N, K, stream);
  return launch_skinny_nt<8, MODE, OutT>(x, ldx, w, o, M, N, K, stream);
}

}  // namespace ms

using namespace ms;

// X [M, K] bfloat16 (mode 0) or gate/up [M, 2K] bfloat16 (mode 1: X = silu(gate) * up); W [N, K] bfloat16;
// out [M, N] bfloat16 (out_dtype 1) or float32 (0).  M <= 64, K a multiple of 8.
MS_EXPORT int ms_gemm_skinny(const void* X, int mode, const void* W, void* out, int out_dtype, int M, int N, int K,
                             cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(M <= 64, "gemm_skinny: %d rows exceed 64", M);
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_skinny: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(mode == MODE_PLAIN || mode == MODE_SILU_MUL, "gemm_skinny: unknown mode %d", mode);
  const int ldx = mode == MODE_PLAIN ? K : 2 * K;
  if (mode == MODE_PLAIN) {
    if (out_dtype == MS_BF16) return launch_skinny<MODE_PLAIN, __nv_bfloat16>(X, ldx, W, out, M, N, K, stream);
    if (out_dtype == MS_F32) return launch_skinny<MODE_PLAIN, float>(X, ldx, W, out, M, N, K, stream);
  } else {
    if (out_dtype == MS_BF16) return launch_skinny<MODE_SILU_MUL, __nv_bfloat16>(X, ldx, W, out, M, N, K, stream);
    if (out_dtype == MS_F32) return launch_skinny<MODE_SILU_MUL, float>(X, ldx, W, out, M, N, K, stream);
  }
  MS_FAIL("gemm_skinny: unknown output type code %d", out_dtype);
}
