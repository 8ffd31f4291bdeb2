// Paged grouped-query attention, general form: any head size up to 512, any page
// size, any mix of prompt portions and decoded tokens, optional sliding window.
// float32 arithmetic throughout (scores, softmax, weighted sum); storage float32 or
// bfloat16.  This is the kernel of the float32 path and the fallback of the bfloat16
// path for sizes its tensor-core kernels do not take.
//
// One thread block of four warps per (token, query head).  Keys are walked in blocks
// of 32 that start at absolute key index 0; warp w takes blocks w, w+4, ...; in a block
// each lane scores one key (a serial dot product over the head), the warp updates its
// running maximum and sum, then each lane accumulates its output lanes over the 32
// values.  The four partial results are merged in warp order.  The order of every sum
// therefore depends only on the token's own position, not on the batch, the portion or
// the pages it lies in.
//
// Two optional changes of a score s between query position p and key position j, applied in this
// order before the softmax: a soft cap, s = cap * tanh(s / cap); and a bias that grows with the
// distance, s += slope[head] * (j - p) (one slope per query head; zero at the query's own key).
#include "common.cuh"

namespace ms {

constexpr int kAttnWarps = 4;
constexpr int kMaxLanesPerThread = 16;  // head size up to 512

// Dot product of a float32 vector in shared memory with one stored row, summed in index
// order; rows are read 16 bytes at a time when the head size allows it.
__device__ __forceinline__ float dot_row(const float* q_s, const float* row, int d) {
  float dot = 0.f;
  if ((d & 3) == 0) {
    for (int c = 0; c < d; c += 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + c);
      dot += q_s[c] * v.x;
      dot += q_s[c + 1] * v.y;
      dot += q_s[c + 2] * v.z;
      dot += q_s[c + 3] * v.w;
    }
  } else {
    for (int c = 0; c < d; ++c) dot += q_s[c] * row[c];
  }
  return dot;
}

__device__ __forceinline__ float dot_row(const float* q_s, const __nv_bfloat16* row, int d) {
  float dot = 0.f;
  if ((d & 7) == 0) {
    for (int c = 0; c < d; c += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(pairs[i]);
        dot += q_s[c + 2 * i] * f.x;
        dot += q_s[c + 2 * i + 1] * f.y;
      }
    }
  } else {
    for (int c = 0; c < d; ++c) dot += q_s[c] * __bfloat162float(row[c]);
  }
  return dot;
}

template <typename T>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                               const T* __restrict__ v_pool, const int* __restrict__ block_tables,
                                               int table_stride, const int* __restrict__ request_of_token,
                                               const int* __restrict__ positions, int page_size, int n_q, int n_kv,
                                               int d, float scale, int window, float softcap,
                                               const float* __restrict__ bias_slopes, T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float smem[];
  float* q_s = smem;                                  // [d]
  float* part_acc = smem + d;                         // [warps][d]
  float* part_m = part_acc + kAttnWarps * d;          // [warps]
  float* part_l = part_m + kAttnWarps;                // [warps]

  const int token = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_head = head / (n_q / n_kv);
  const int pos = positions[token];
  const int* table = block_tables + (size_t)request_of_token[token] * table_stride;
  const T* q_row = q + ((size_t)token * n_q + head) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) q_s[c] = to_float(q_row[c]) * scale;
  __syncthreads();

  const float slope = bias_slopes ? bias_slopes[head] : 0.f;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int last_key = pos;  // inclusive
  float m = -INFINITY, l = 0.f;
  float acc[kMaxLanesPerThread];
#pragma unroll
  for (int i = 0; i < kMaxLanesPerThread; ++i) acc[i] = 0.f;

  const int first_block = first_key / 32, last_block = last_key / 32;
  for (int block = first_block + ((warp - first_block % kAttnWarps + kAttnWarps) % kAttnWarps); block <= last_block;
       block += kAttnWarps) {
    const int key = block * 32 + lane;
    const bool valid = key >= first_key && key <= last_key;
    float score = -INFINITY;
    size_t row_offset = 0;
    if (valid) {
      const int page = table[key / page_size];
      row_offset = (((size_t)page * n_kv + kv_head) * page_size + key % page_size) * d;
      score = dot_row(q_s, k_pool + row_offset, d);
      if (softcap > 0.f) score = softcap * tanhf(score / softcap);
      score += slope * (float)(key - pos);
    }
    const float block_max = warp_max(score);
    const float new_m = fmaxf(m, block_max);       // finite: every block holds at least one valid key
    const float correction = expf(m - new_m);      // m == -inf on the first block gives 0
    const float p = valid ? expf(score - new_m) : 0.f;
    l = l * correction + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int i = 0; i < kMaxLanesPerThread; ++i) acc[i] *= correction;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off_j = __shfl_sync(0xffffffffu, (unsigned long long)row_offset, j);
      if (pj == 0.f) continue;   // uniform across the warp
      const T* v_row = v_pool + off_j;
#pragma unroll
      for (int i = 0; i < kMaxLanesPerThread; ++i) {
        const int c = lane + 32 * i;
        if (c < d) acc[i] += pj * to_float(v_row[c]);
      }
    }
  }

  if (lane == 0) {
    part_m[warp] = m;
    part_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < kMaxLanesPerThread; ++i) {
    const int c = lane + 32 * i;
    if (c < d) part_acc[warp * d + c] = acc[i];
  }
  __syncthreads();
  float m_all = -INFINITY;
  for (int w = 0; w < kAttnWarps; ++w) m_all = fmaxf(m_all, part_m[w]);
  float l_all = 0.f;
  for (int w = 0; w < kAttnWarps; ++w) l_all += part_m[w] == -INFINITY ? 0.f : part_l[w] * expf(part_m[w] - m_all);
  T* out_row = out + ((size_t)token * n_q + head) * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float sum = 0.f;
    for (int w = 0; w < kAttnWarps; ++w)
      if (part_m[w] != -INFINITY) sum += part_acc[w * d + c] * expf(part_m[w] - m_all);
    out_row[c] = from_float<T>(sum / l_all);
  }
}

}  // namespace ms

using namespace ms;

// q [n_tokens, n_q, d]; pools of one layer [pages, n_kv, page_size, d]; block_tables
// [requests, table_stride]; request_of_token, positions [n_tokens]; out [n_tokens, n_q, d].
// The keys of a token are positions max(0, pos - window + 1) .. pos of its own request
// (window <= 0: no window); they must already be in the pool.  softcap <= 0: no soft cap; bias_slopes
// [n_q] float32 or null.
MS_EXPORT int ms_paged_attention_generic(const void* q, int dtype, const void* k_pool, const void* v_pool,
                                         const int* block_tables, int table_stride, const int* request_of_token,
                                         const int* positions, int page_size, int n_q, int n_kv, int d, float scale,
                                         int window, float softcap, const float* bias_slopes, void* out, int n_tokens,
                                         cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(d > 0 && d <= 32 * kMaxLanesPerThread, "paged_attention: head size %d outside 1..%d", d,
             32 * kMaxLanesPerThread);
  MS_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "paged_attention: %d query heads are not a multiple of %d key/value heads",
             n_q, n_kv);
  MS_REQUIRE(page_size > 0, "paged_attention: page size must be positive, got %d", page_size);
  MS_REQUIRE(n_q <= 65535, "paged_attention: %d query heads exceed 65535", n_q);
  const size_t smem = (size_t)(d + kAttnWarps * d + 2 * kAttnWarps) * sizeof(float);
  dim3 grid(n_tokens, n_q);
  if (dtype == MS_F32) {
    ms::launch(paged_attention_generic_kernel<float>, grid, kAttnWarps * 32, smem, stream, 
        (const float*)q, (const float*)k_pool, (const float*)v_pool, block_tables, table_stride, request_of_token,
        positions, page_size, n_q, n_kv, d, scale, window, softcap, bias_slopes, (float*)out);
  } else if (dtype == MS_BF16) {
    ms::launch(paged_attention_generic_kernel<__nv_bfloat16>, grid, kAttnWarps * 32, smem, stream, 
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, block_tables,
        table_stride, request_of_token, positions, page_size, n_q, n_kv, d, scale, window, softcap, bias_slopes,
        (__nv_bfloat16*)out);
  } else {
    MS_FAIL("paged_attention: unknown element type code %d", dtype);
  }
  MS_CHECK_LAUNCH("paged_attention_generic");
  return 0;
}
