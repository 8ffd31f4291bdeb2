// Memory-bound kernels between the matrix products: embedding, residual add fused
// with RMSNorm, rotation tables, per-head norm + rotation + paged cache append, and
// the gated activation.  All arithmetic is float32; storage is float32 or bfloat16.
#include "common.cuh"
#include "elementwise_vec.cuh"

namespace ms {

// ---------------------------------------------------------------- embedding
// out[n, :] = scale * float(table[token[n], :]); the residual stream is float32.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, float scale) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t row = blockIdx.x;
  const T* src = table + (size_t)tokens[row] * hidden;
  float* dst = out + row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = scale * to_float(src[c]);
}

// ---------------------------------------------------------------- logit transform
// x = scale * x, then (cap > 0) x = cap * tanh(x / cap), in place on float32.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t total, float scale, float cap) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v = scale * x[i];
  if (cap > 0.f) v = cap * tanhf(v / cap);
  x[i] = v;
}

// ---------------------------------------------------------------- residual add + RMSNorm
// For output row k (source row r = rows ? rows[k] : k):
//   x = residual[r] + delta[r]            (float32; written back to residual unless gathered)
//   out[k] = weight * x * rsqrt(mean(x^2) + eps)   rounded once to T
// `delta` may be null (no add).  The weight keeps its stored type (float32 or bfloat16).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const void* __restrict__ weight, int weight_dtype,
                                   const int* __restrict__ rows, T* __restrict__ out,
                                   int hidden, float eps) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t k = blockIdx.x;
  const size_t r = rows ? (size_t)rows[k] : k;
  float* res = residual + r * hidden;
  const T* del = delta ? delta + r * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (delta != nullptr);
  float sum_sq = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = res[c];
    if (del) x += to_float(del[c]);
    if (write_back) res[c] = x;
    sum_sq += x * x;
  }
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* dst = out + k * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = res[c];
    if (del && !write_back) x += to_float(del[c]);
    dst[c] = from_float<T>(load_as_float(weight, weight_dtype, c) * (x * inv));
  }
}

// ---------------------------------------------------------------- plain RMSNorm on T rows
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const void* __restrict__ weight, int weight_dtype,
                               T* __restrict__ out, int hidden, float eps) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const T* src = x + (size_t)blockIdx.x * hidden;
  float sum_sq = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = to_float(src[c]);
    sum_sq += v * v;
  }
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* dst = out + (size_t)blockIdx.x * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    dst[c] = from_float<T>(load_as_float(weight, weight_dtype, c) * (to_float(src[c]) * inv));
}

// ---------------------------------------------------------------- rotation tables
// cos_sin[n, j] = (cos, sin)(float(position[n]) * inv_freq[j]) for j < half, in float32.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int n_tokens, int half) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * half) return;
  const int n = i / half, j = i % half;
  const float angle = (float)positions[n] * inv_freq[j];
  float s, c;
  sincosf(angle, &s, &c);
  cos_sin[i] = make_float2(c, s);
}

// ---------------------------------------------------------------- q/k norm + rotation + cache append
// One warp per (token, head) of the fused projection output qkv[n, (nq + 2 nkv) * d].
//   q heads: optional RMSNorm over d, rotation, written to q_out[n, head, :]
//   k heads: optional RMSNorm over d, rotation, written to the key pool at the token's slot
//   v heads: copied to the value pool at the token's slot
// Rotation acts on the first `rotary_dim` lanes of a head: half-split pairs (j, j + rotary_dim/2)
// or interleaved pairs (2j, 2j+1); `cos_sin` null means no rotation.
// Pool layout of one layer: [page, kv_head, page_size, d]; slot = page * page_size + offset;
// a negative slot skips the write.
template <typename T>
__global__ void qk_norm_rope_append_kernel(const T* __restrict__ qkv, const int* __restrict__ slots,
                                           const void* __restrict__ q_weight, const void* __restrict__ k_weight,
                                           int weight_dtype, float eps, const float2* __restrict__ cos_sin,
                                           int rotary_dim, int interleaved, T* __restrict__ k_pool,
                                           T* __restrict__ v_pool, int page_size, int n_q, int n_kv, int d,
                                           T* __restrict__ q_out, int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float smem[];
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = n_q + 2 * n_kv;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)n_tokens * heads) return;
  const int n = (int)(item / heads), head = (int)(item % heads);
  const T* src = qkv + ((size_t)n * heads + head) * d;
  float* x = smem + warp * d;

  T* dst;
  const void* weight = nullptr;
  bool rotate = false;
  if (head < n_q) {
    dst = q_out + ((size_t)n * n_q + head) * d;
    weight = q_weight;
    rotate = cos_sin != nullptr;
  } else {
    const int slot = slots[n];
    if (slot < 0) return;
    const int page = slot / page_size, offset = slot % page_size;
    const bool is_key = head < n_q + n_kv;
    const int kv_head = is_key ? head - n_q : head - n_q - n_kv;
    T* pool = is_key ? k_pool : v_pool;
    dst = pool + (((size_t)page * n_kv + kv_head) * page_size + offset) * d;
    if (is_key) {
      weight = k_weight;
      rotate = cos_sin != nullptr;
    } else {
      for (int c = lane; c < d; c += 32) dst[c] = src[c];
      return;
    }
  }

  float sum_sq = 0.f;
  for (int c = lane; c < d; c += 32) {
    const float v = to_float(src[c]);
    x[c] = v;
    sum_sq += v * v;
  }
  float inv = 1.f;
  if (weight) {
    sum_sq = warp_sum(sum_sq);
    inv = 1.0f / sqrtf(sum_sq / (float)d + eps);
  }
  __syncwarp();
  const int half = rotary_dim >> 1;
  const float2* table = cos_sin ? cos_sin + (size_t)n * half : nullptr;
  for (int c = lane; c < d; c += 32) {
    float v = x[c] * inv;
    if (weight) v *= load_as_float(weight, weight_dtype, c);
    if (rotate && c < rotary_dim) {
      int partner, j;
      float sign;
      if (interleaved) {
        j = c >> 1;
        partner = c ^ 1;
        sign = (c & 1) ? 1.f : -1.f;
      } else {
        j = c < half ? c : c - half;
        partner = c < half ? c + half : c - half;
        sign = c < half ? -1.f : 1.f;
      }
      float p = x[partner] * inv;
      if (weight) p *= load_as_float(weight, weight_dtype, partner);
      const float2 cs = table[j];
      v = v * cs.x + sign * p * cs.y;
    }
    dst[c] = from_float<T>(v);
  }
}

// ---------------------------------------------------------------- gated activation
// out[n, c] = silu(gate_up[n, c]) * gate_up[n, inter + c]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t n = i / inter;
  const int c = (int)(i % inter);
  const float g = to_float(gate_up[n * 2 * inter + c]);
  const float u = to_float(gate_up[n * 2 * inter + inter + c]);
  out[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

}  // namespace ms

using namespace ms;

#define MS_DISPATCH(dtype, ...)                                  \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

MS_EXPORT int ms_embedding(const int* tokens, const void* table, int dtype, float* out, int n_tokens, int hidden,
                           float scale, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(hidden > 0, "embedding: hidden size must be positive, got %d", hidden);
  MS_DISPATCH(dtype, (ms::launch(embedding_kernel<T>, n_tokens, 256, 0, stream, tokens, (const T*)table, out, hidden, scale)));
  MS_CHECK_LAUNCH("embedding");
  return 0;
}

// x [total] float32 in place: x = scale * x, then, if cap > 0, x = cap * tanh(x / cap).
MS_EXPORT int ms_scale_softcap(float* x, long long total, float scale, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "scale_softcap: %lld elements in one launch is too many", total);
  ms::launch(scale_softcap_kernel, (unsigned)blocks, 256, 0, stream, x, (size_t)total, scale, cap);
  MS_CHECK_LAUNCH("scale_softcap");
  return 0;
}

MS_EXPORT int ms_add_rmsnorm(float* residual, const void* delta, int dtype, const void* weight, int weight_dtype,
                             const int* rows, void* out, int n_out, int hidden, float eps, cudaStream_t stream) {
  if (n_out == 0) return 0;
  MS_REQUIRE(hidden > 0, "add_rmsnorm: hidden size must be positive, got %d", hidden);
  if (hidden % 8 == 0 && hidden <= 8192) {
    const int groups = hidden / 8;
    const int threads = groups >= 256 ? 256 : ((groups + 31) / 32) * 32;
    const int chunks = (groups + threads - 1) / threads;
#define MS_ADD_RMSNORM_VEC(C)                                                                                     \
  MS_DISPATCH(dtype, (ms::launch(add_rmsnorm_vec_kernel<T, C>, n_out, threads, 0, stream, residual, (const T*)delta, weight, \
                                                                               weight_dtype, rows, (T*)out, hidden, eps)))
    if (chunks == 1) { MS_ADD_RMSNORM_VEC(1); } else if (chunks == 2) { MS_ADD_RMSNORM_VEC(2); } else { MS_ADD_RMSNORM_VEC(4); }
#undef MS_ADD_RMSNORM_VEC
    MS_CHECK_LAUNCH("add_rmsnorm");
    return 0;
  }
  const int threads = hidden >= 1024 ? 256 : 128;
  MS_DISPATCH(dtype, (ms::launch(add_rmsnorm_kernel<T>, n_out, threads, 0, stream, residual, (const T*)delta, weight,
                                                                         weight_dtype, rows, (T*)out, hidden, eps)));
  MS_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}

MS_EXPORT int ms_rmsnorm(const void* x, int dtype, const void* weight, int weight_dtype, void* out, int n_rows,
                         int hidden, float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  MS_REQUIRE(hidden > 0, "rmsnorm: size must be positive, got %d", hidden);
  const int threads = hidden >= 1024 ? 256 : (hidden >= 128 ? 128 : 32);
  MS_DISPATCH(dtype, (ms::launch(rmsnorm_kernel<T>, n_rows, threads, 0, stream, (const T*)x, weight, weight_dtype, (T*)out,
                                                                      hidden, eps)));
  MS_CHECK_LAUNCH("rmsnorm");
  return 0;
}

MS_EXPORT int ms_rope_table(const int* positions, const float* inv_freq, float* cos_sin, int n_tokens, int half,
                            cudaStream_t stream) {
  if (n_tokens == 0 || half == 0) return 0;
  const int total = n_tokens * half;
  ms::launch(rope_table_kernel, (total + 255) / 256, 256, 0, stream, positions, inv_freq, (float2*)cos_sin, n_tokens, half);
  MS_CHECK_LAUNCH("rope_table");
  return 0;
}

MS_EXPORT int ms_qk_norm_rope_append(const void* qkv, int dtype, const int* slots, const void* q_weight,
                                     const void* k_weight, int weight_dtype, float eps, const float* cos_sin,
                                     int rotary_dim, int interleaved, void* k_pool, void* v_pool, int page_size,
                                     int n_q, int n_kv, int d, void* q_out, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(d > 0 && d <= 1024, "qk_norm_rope_append: head size %d outside 1..1024", d);
  MS_REQUIRE(rotary_dim >= 0 && rotary_dim <= d && rotary_dim % 2 == 0,
             "qk_norm_rope_append: rotary size %d must be even and at most the head size %d", rotary_dim, d);
  MS_REQUIRE(page_size > 0, "qk_norm_rope_append: page size must be positive, got %d", page_size);
  const int warps = 4;
  const long long items = (long long)n_tokens * (n_q + 2 * n_kv);
  const long long blocks = (items + warps - 1) / warps;
  MS_REQUIRE(blocks < 2147483647LL, "qk_norm_rope_append: %lld heads in one launch is too many", items);
  const bool vector_ok = d % 8 == 0 && d <= 256 && (cos_sin == nullptr || interleaved || rotary_dim % 16 == 0);
  if (vector_ok) {
    const int lanes_needed = d / 8;
    const bool pow2 = (lanes_needed & (lanes_needed - 1)) == 0;
    const int lanes = pow2 ? lanes_needed : 32;            // lanes per head
    const int heads_per_warp = 32 / lanes;
    const long long warps_needed = (items + heads_per_warp - 1) / heads_per_warp;
    const long long vec_blocks = (warps_needed + warps - 1) / warps;
    // half-split rotation over the whole head: each lane holds an element group and its partner group
    const bool pairs = cos_sin != nullptr && !interleaved && rotary_dim == d && pow2;
#define MS_ROPE_VEC(L, P)                                                                                              \
  MS_DISPATCH(dtype, (ms::launch(qk_norm_rope_append_vec_kernel<T, L, P>, (unsigned)vec_blocks, warps * 32, 0, stream, \
                                 (const T*)qkv, slots, q_weight, k_weight, weight_dtype, eps, cos_sin, rotary_dim,     \
                                 interleaved, (T*)k_pool, (T*)v_pool, page_size, n_q, n_kv, d, (T*)q_out, n_tokens)))
    if (pairs) {
      if (lanes == 2) { MS_ROPE_VEC(2, true); } else if (lanes == 4) { MS_ROPE_VEC(4, true); }
      else if (lanes == 8) { MS_ROPE_VEC(8, true); } else if (lanes == 16) { MS_ROPE_VEC(16, true); }
      else { MS_ROPE_VEC(32, true); }
    } else {
      if (lanes == 2) { MS_ROPE_VEC(2, false); } else if (lanes == 4) { MS_ROPE_VEC(4, false); }
      else if (lanes == 8) { MS_ROPE_VEC(8, false); } else if (lanes == 16) { MS_ROPE_VEC(16, false); }
      else { MS_ROPE_VEC(32, false); }
    }
#undef MS_ROPE_VEC
    MS_CHECK_LAUNCH("qk_norm_rope_append");
    return 0;
  }
  const size_t smem = (size_t)warps * d * sizeof(float);
  MS_DISPATCH(dtype, (ms::launch(qk_norm_rope_append_kernel<T>, (unsigned)blocks, warps * 32, smem, stream, 
                         (const T*)qkv, slots, q_weight, k_weight, weight_dtype, eps, (const float2*)cos_sin,
                         rotary_dim, interleaved, (T*)k_pool, (T*)v_pool, page_size, n_q, n_kv, d, (T*)q_out,
                         n_tokens)));
  MS_CHECK_LAUNCH("qk_norm_rope_append");
  return 0;
}

// paired != 0: gate and up columns alternate in blocks of eight (inter must be a multiple of 8 then).
MS_EXPORT int ms_silu_mul(const void* gate_up, int dtype, void* out, int n_tokens, int inter, int paired, cudaStream_t stream) {
  const size_t total = (size_t)n_tokens * inter;
  if (total == 0) return 0;
  MS_REQUIRE(!paired || inter % 8 == 0, "silu_mul: paired columns need a multiple of 8 features, not %d", inter);
  if (inter % 8 == 0) {
    const size_t total8 = total / 8;
    const size_t blocks8 = (total8 + 255) / 256;
    MS_REQUIRE(blocks8 < 2147483647ULL, "silu_mul: %zu elements in one launch is too many", total);
    MS_DISPATCH(dtype, (ms::launch(silu_mul_vec_kernel<T>, (unsigned)blocks8, 256, 0, stream, (const T*)gate_up, (T*)out, inter,
                                                                                    total8, paired)));
    MS_CHECK_LAUNCH("silu_mul");
    return 0;
  }
  const size_t blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647ULL, "silu_mul: %zu elements in one launch is too many", total);
  MS_DISPATCH(dtype, (ms::launch(silu_mul_kernel<T>, (unsigned)blocks, 256, 0, stream, (const T*)gate_up, (T*)out, inter,
                                                                             total)));
  MS_CHECK_LAUNCH("silu_mul");
  return 0;
}
