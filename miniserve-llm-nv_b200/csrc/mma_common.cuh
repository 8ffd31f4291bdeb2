// What the mma.sync attention kernels share: asynchronous 16-byte copies, ldmatrix and mma.m16n8k16 wrappers,
// the swizzled layout of their shared-memory tiles, and the kernel that merges the splits of the keys
// (attention_mma.cu, attention_decode.cu).
#pragma once

#include "common.cuh"

namespace ms {

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
  const int bytes = valid ? 16 : 0;   // zero-fills the 16 bytes when not valid
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Shared-memory tiles are [rows][D] bfloat16 with the 16-byte chunks of a row XOR-swizzled by
// the row index, so that ldmatrix reads eight rows without bank conflicts.
// A row of D elements has D / 8 chunks; the XOR mask never leaves the row: rows of 128 bytes or
// more use the low three row bits, 64-byte rows (D = 32) the row bits 1..2, so that in both cases
// eight consecutive rows land in eight different 16-byte bank groups.
template <int D> __device__ __forceinline__ __nv_bfloat16* tile_ptr(__nv_bfloat16* base, int row, int chunk) {
  static_assert(D % 32 == 0, "head size must be a multiple of 32 for this kernel");
  constexpr int CHUNKS = D / 8;
  const int mask = CHUNKS >= 8 ? (row & 7) : ((row >> 1) & (CHUNKS - 1));
  return base + row * D + ((chunk ^ mask) << 3);
}

// Merges the splits of one (token, head): out = sum_s w_s O_s / sum_s w_s with w_s = 2^(lse_s - max lse).
// One block of four warps per (token, head).  Warp w takes the splits w, w + 4, ... (at most 64 splits, so
// at most 16 each) and requests all of their partial results at once, before it reads the splits' weights:
// the merge then costs one trip to the L2 cache, not one per group of splits.  Lane s of every warp holds the
// weight of split s and s + 32; the four warps' sums are added in warp order through shared memory.
// The same merge with all of up to 64 splits requested at once (sixteen per warp): for steps of one or two requests,
// whose keys are cut into 32 to 64 splits; launch_attention_combine chooses.
template <int D>
__global__ void __launch_bounds__(128)
attention_combine_all_at_once_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                         __nv_bfloat16* __restrict__ out, int num_splits, int n_items) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float warp_acc[4][D];
  const int item = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* base = part_o + (size_t)item * num_splits * D;
  float v[16][D / 32];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int s = warp + 4 * j;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) v[j][i] = s < num_splits ? __ldcg(base + (size_t)s * D + lane + 32 * i) : 0.f;
  }
  const float* lse = part_lse + (size_t)item * num_splits;
  const float lse_a = lane < num_splits ? __ldcg(lse + lane) : -INFINITY;
  const float lse_b = lane + 32 < num_splits ? __ldcg(lse + lane + 32) : -INFINITY;
  const float m = warp_max(fmaxf(lse_a, lse_b));
  const float w_a = lse_a == -INFINITY ? 0.f : exp2f(lse_a - m);
  const float w_b = lse_b == -INFINITY ? 0.f : exp2f(lse_b - m);
  const float total = warp_sum(w_a + w_b);
  float acc[D / 32] = {};
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int s = warp + 4 * j;                      // (a split without keys has weight 0: its buffer is not added)
    const float w = __shfl_sync(0xffffffffu, s < 32 ? w_a : w_b, s & 31);
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += (s < num_splits && w != 0.f) ? w * v[j][i] : 0.f;
  }
#pragma unroll
  for (int i = 0; i < D / 32; ++i) warp_acc[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  if (warp == 0) {
    const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int c = lane + 32 * i;
      const float sum = ((warp_acc[0][c] + warp_acc[1][c]) + warp_acc[2][c]) + warp_acc[3][c];
      out[(size_t)item * D + c] = __float2bfloat16_rn(sum * inv);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(128)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                         __nv_bfloat16* __restrict__ out, int num_splits, int n_items) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float warp_acc[4][D];
  const int item = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* base = part_o + (size_t)item * num_splits * D;
  // This warp's splits (warp, warp + 4, ...) sixteen at a time: the first sixteen are requested before anything
  // else; more are fetched only if there are more (the loop is not unrolled over all 64 possible splits: the kernel
  // runs for three microseconds, and instructions that do nothing still have to be fetched).
  float v[4][D / 32], ahead[4][D / 32];
  auto fetch = [&](float (&to)[4][D / 32], int j0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int s = warp + 4 * (j0 + j);
#pragma unroll
      for (int i = 0; i < D / 32; ++i) to[j][i] = s < num_splits ? __ldcg(base + (size_t)s * D + lane + 32 * i) : 0.f;
    }
  };
  fetch(v, 0);
  const float* lse = part_lse + (size_t)item * num_splits;
  const float lse_a = lane < num_splits ? __ldcg(lse + lane) : -INFINITY;
  const float lse_b = lane + 32 < num_splits ? __ldcg(lse + lane + 32) : -INFINITY;
  const float m = warp_max(fmaxf(lse_a, lse_b));
  const float w_a = lse_a == -INFINITY ? 0.f : exp2f(lse_a - m);
  const float w_b = lse_b == -INFINITY ? 0.f : exp2f(lse_b - m);
  const float total = warp_sum(w_a + w_b);
  float acc[D / 32] = {};
  for (int j0 = 0;;) {
    const bool more = j0 + 4 < 16 && 4 * (j0 + 4) < num_splits;
    if (more) fetch(ahead, j0 + 4);                  // on their way while these are added
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int s = warp + 4 * (j0 + j);             // (a split without keys has weight 0: its buffer is not added)
      const float w = __shfl_sync(0xffffffffu, s < 32 ? w_a : w_b, s & 31);
#pragma unroll
      for (int i = 0; i < D / 32; ++i) acc[i] += (s < num_splits && w != 0.f) ? w * v[j][i] : 0.f;
    }
    if (!more) break;
    j0 += 4;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < D / 32; ++i) v[j][i] = ahead[j][i];
  }
#pragma unroll
  for (int i = 0; i < D / 32; ++i) warp_acc[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  if (warp == 0) {
    const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int c = lane + 32 * i;
      const float sum = ((warp_acc[0][c] + warp_acc[1][c]) + warp_acc[2][c]) + warp_acc[3][c];
      out[(size_t)item * D + c] = __float2bfloat16_rn(sum * inv);
    }
  }
}

// Sixteen splits or fewer: the kernel that fetches sixteen at a time and has no code for the rest on its path.
template <int D>
inline void launch_attention_combine(const float* part_o, const float* part_lse, __nv_bfloat16* out, int num_splits,
                                     int items, cudaStream_t stream) {
  if (num_splits > 16)
    ms::launch(attention_combine_all_at_once_kernel<D>, items, 128, 0, stream, part_o, part_lse, out, num_splits, items);
  else
    ms::launch(attention_combine_kernel<D>, items, 128, 0, stream, part_o, part_lse, out, num_splits, items);
}

}  // namespace ms
