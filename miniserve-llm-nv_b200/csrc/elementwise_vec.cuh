// 16-byte-vectorised forms of the memory-bound kernels, used when the row sizes are
// multiples of eight elements (rows then start on 16-byte boundaries).  Same arithmetic as
// the scalar forms in elementwise.cu: float32 inside, one rounding at the store.
#pragma once

#include "common.cuh"

namespace ms {

// Eight consecutive elements as floats, whatever the stored type.
struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8(const float* p) {
  Vec8 r;
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
  r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
  return r;
}

__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* p) {
  Vec8 r;
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(pairs[i]);
    r.v[2 * i] = f.x;
    r.v[2 * i + 1] = f.y;
  }
  return r;
}

__device__ __forceinline__ Vec8 load8_any(const void* p, int dtype, size_t index) {
  return dtype == MS_F32 ? load8(reinterpret_cast<const float*>(p) + index)
                         : load8(reinterpret_cast<const __nv_bfloat16*>(p) + index);
}

__device__ __forceinline__ void store8(float* p, const Vec8& x) {
  *reinterpret_cast<float4*>(p) = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(x.v[4], x.v[5], x.v[6], x.v[7]);
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const Vec8& x) {
  uint4 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(x.v[2 * i], x.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Four consecutive elements into v[offset .. offset + 3].
__device__ __forceinline__ void load4(const float* p, Vec8& r, int offset) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  r.v[offset] = a.x; r.v[offset + 1] = a.y; r.v[offset + 2] = a.z; r.v[offset + 3] = a.w;
}

__device__ __forceinline__ void load4(const __nv_bfloat16* p, Vec8& r, int offset) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]);
  r.v[offset] = a.x; r.v[offset + 1] = a.y; r.v[offset + 2] = b.x; r.v[offset + 3] = b.y;
}

__device__ __forceinline__ void load4_any(const void* p, int dtype, size_t index, Vec8& r, int offset) {
  if (dtype == MS_F32) load4(reinterpret_cast<const float*>(p) + index, r, offset);
  else load4(reinterpret_cast<const __nv_bfloat16*>(p) + index, r, offset);
}

__device__ __forceinline__ void store4(float* p, const Vec8& x, int offset) {
  *reinterpret_cast<float4*>(p) = make_float4(x.v[offset], x.v[offset + 1], x.v[offset + 2], x.v[offset + 3]);
}

__device__ __forceinline__ void store4(__nv_bfloat16* p, const Vec8& x, int offset) {
  uint2 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
  pairs[0] = __floats2bfloat162_rn(x.v[offset], x.v[offset + 1]);
  pairs[1] = __floats2bfloat162_rn(x.v[offset + 2], x.v[offset + 3]);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row; each thread keeps up to CHUNKS groups of eight elements in registers,
// so the row is read once.  Requires hidden % 8 == 0 and hidden <= 8 * blockDim.x * CHUNKS.
template <typename T, int CHUNKS>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                       const void* __restrict__ weight, int weight_dtype,
                                       const int* __restrict__ rows, T* __restrict__ out, int hidden, float eps) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t k = blockIdx.x;
  const size_t r = rows ? (size_t)rows[k] : k;
  float* res = residual + r * hidden;
  const T* del = delta ? delta + r * hidden : nullptr;
  const bool write_back = (rows == nullptr) && (delta != nullptr);
  Vec8 x[CHUNKS];
  float sum_sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      x[i] = load8(res + c);
      if (del) {
        const Vec8 d = load8(del + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[i].v[e] += d.v[e];
        if (write_back) store8(res + c, x[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sum_sq += x[i].v[e] * x[i].v[e];
    }
  }
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* dst = out + k * hidden;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = (i * blockDim.x + threadIdx.x) * 8;
    if (c < hidden) {
      const Vec8 w = load8_any(weight, weight_dtype, c);
      Vec8 y;
#pragma unroll
      for (int e = 0; e < 8; ++e) y.v[e] = w.v[e] * (x[i].v[e] * inv);
      store8(dst + c, y);
    }
  }
}

// ---------------------------------------------------------------- q/k norm + rotation + cache append
// A group of d / 8 lanes per (token, head); lane l of the group holds elements 8l .. 8l+7 of the head.
// LANES is the group size: 32 / LANES heads share a warp when d / 8 is a power of two, else a head has
// the warp to itself (LANES = 32, lanes beyond d / 8 idle).  d <= 256, d % 8 == 0.  Half-split rotation
// needs rotary_dim % 16 == 0 so that an element's partner sits at the same place in another lane of the
// group; interleaved pairs sit within a lane.
// PAIRS (half-split rotation over the whole head, the usual case): lane l holds elements 4l .. 4l+3 and
// their partners d/2 + 4l .. d/2 + 4l+3 instead, so the rotation needs no exchange between lanes (the
// kernel is bound by the shuffles and loads it issues, not by arithmetic or bandwidth).
template <typename T, int LANES, bool PAIRS = false>
__global__ void qk_norm_rope_append_vec_kernel(const T* __restrict__ qkv, const int* __restrict__ slots,
                                               const void* __restrict__ q_weight, const void* __restrict__ k_weight,
                                               int weight_dtype, float eps, const float* __restrict__ cos_sin,
                                               int rotary_dim, int interleaved, T* __restrict__ k_pool,
                                               T* __restrict__ v_pool, int page_size, int n_q, int n_kv, int d,
                                               T* __restrict__ q_out, int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  constexpr int HEADS_PER_WARP = 32 / LANES;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LANES, sub_lane = lane % LANES;
  const int heads = n_q + 2 * n_kv;
  const long long total = (long long)n_tokens * heads;
  const long long item = ((long long)blockIdx.x * warps_per_block + warp) * HEADS_PER_WARP + sub;
  // No early exit: the lanes of a warp may serve different heads and all of them take part in the shuffles.
  const bool item_ok = item < total;
  int n = 0, head = 0;
  if (item_ok) {
    if (total <= 0x7fffffffLL) {                       // 32-bit division where it is enough
      n = (int)((unsigned)item / (unsigned)heads);
      head = (int)((unsigned)item % (unsigned)heads);
    } else {
      n = (int)(item / heads);
      head = (int)(item % heads);
    }
  }
  const T* src = qkv + ((size_t)n * heads + head) * d;
  const int c0 = PAIRS ? sub_lane * 4 : sub_lane * 8;      // PAIRS: also elements c0 + d/2 ..
  const int c1 = c0 + (d >> 1);
  bool active = item_ok && (PAIRS ? c0 < (d >> 1) : c0 < d);

  T* dst = nullptr;
  const void* weight = nullptr;
  bool is_value = false;
  if (head < n_q) {
    dst = q_out + ((size_t)n * n_q + head) * d;
    weight = q_weight;
  } else {
    const int slot = item_ok ? slots[n] : -1;
    if (slot < 0) {
      active = false;
    } else {
      const int page = slot / page_size, offset = slot % page_size;
      const bool is_key = head < n_q + n_kv;
      const int kv_head = is_key ? head - n_q : head - n_q - n_kv;
      dst = (is_key ? k_pool : v_pool) + (((size_t)page * n_kv + kv_head) * page_size + offset) * d;
      is_value = !is_key;
      weight = is_key ? k_weight : nullptr;
    }
  }
  const bool rotate = cos_sin != nullptr && !is_value;

  Vec8 x;
#pragma unroll
  for (int e = 0; e < 8; ++e) x.v[e] = 0.f;
  if (active) {
    if (PAIRS) {
      load4(src + c0, x, 0);
      load4(src + c1, x, 4);
    } else {
      x = load8(src + c0);
    }
  }
  {
    float sum_sq = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) sum_sq += x.v[e] * x.v[e];
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) sum_sq += __shfl_xor_sync(0xffffffffu, sum_sq, o);
    if (weight && active) {
      const float inv = 1.0f / sqrtf(sum_sq / (float)d + eps);
      Vec8 w;
      if (PAIRS) {
        load4_any(weight, weight_dtype, c0, w, 0);
        load4_any(weight, weight_dtype, c1, w, 4);
      } else {
        w = load8_any(weight, weight_dtype, c0);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) x.v[e] = x.v[e] * inv * w.v[e];
    }
  }
  if (cos_sin != nullptr) {                                  // uniform: every lane takes part in the shuffles
    const int half = rotary_dim >> 1;
    const float* table = cos_sin + (size_t)n * rotary_dim;       // [half][2] floats
    if (PAIRS) {
      if (rotate && active) {
        const Vec8 cs = load8(table + 2 * c0);                   // (cos, sin) of pairs c0 .. c0+3
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float c = cs.v[2 * e], sn = cs.v[2 * e + 1];
          const float a = x.v[e], b = x.v[4 + e];
          x.v[e] = a * c - b * sn;
          x.v[4 + e] = b * c + a * sn;
        }
      }
    } else if (interleaved) {
      if (rotate && active && c0 < rotary_dim) {
        const Vec8 cs = load8(table + c0);                       // (cos, sin) of pairs c0/2 .. c0/2+3
        Vec8 y;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float c = cs.v[2 * p], s = cs.v[2 * p + 1];
          y.v[2 * p] = x.v[2 * p] * c - x.v[2 * p + 1] * s;
          y.v[2 * p + 1] = x.v[2 * p + 1] * c + x.v[2 * p] * s;
        }
        x = y;
      }
    } else {
      const int lanes_half = half >> 3;                          // lanes that hold one half of the rotary part
      const bool first = c0 < half;
      const int partner_sub_lane = first ? sub_lane + lanes_half : sub_lane - lanes_half;
      const int partner_lane = sub * LANES + (partner_sub_lane & (LANES - 1));
      Vec8 partner;
#pragma unroll
      for (int e = 0; e < 8; ++e) partner.v[e] = __shfl_sync(0xffffffffu, x.v[e], partner_lane);
      if (rotate && active && c0 < rotary_dim) {
        const int j0 = first ? c0 : c0 - half;
        const Vec8 cs_a = load8(table + 2 * j0);
        const Vec8 cs_b = load8(table + 2 * j0 + 8);
        const float sign = first ? -1.f : 1.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float c = e < 4 ? cs_a.v[2 * e] : cs_b.v[2 * (e - 4)];
          const float s = e < 4 ? cs_a.v[2 * e + 1] : cs_b.v[2 * (e - 4) + 1];
          x.v[e] = x.v[e] * c + sign * partner.v[e] * s;
        }
      }
    }
  }
  if (active) {
    if (PAIRS) {
      // (a value passed through float and back is the same value)
      store4(dst + c0, x, 0);
      store4(dst + c1, x, 4);
    } else if (is_value) {
      // values are copied bit for bit
      *reinterpret_cast<uint4*>(dst + c0) = *reinterpret_cast<const uint4*>(src + c0);
      if (sizeof(T) == 4) *reinterpret_cast<uint4*>(dst + c0 + 4) = *reinterpret_cast<const uint4*>(src + c0 + 4);
    } else {
      store8(dst + c0, x);
    }
  }
}

// ---------------------------------------------------------------- gated activation
// Eight outputs per thread; requires inter % 8 == 0.  `paired`: the columns of gate_up come in blocks of
// sixteen, eight gate columns followed by the up columns of the same eight features (the layout that the
// fused product of few rows wants of the weight's rows); else all gate columns precede all up columns.
// silu(g) * u.  With bfloat16 data the exponential and the division are the fast ones (relative error about
// 2^-21, far below the rounding of the result to 8 bits of mantissa); float32 data keeps the accurate ones.
template <typename T>
__device__ __forceinline__ float silu_times(float g, float u) {
  if (sizeof(T) == 2) {
    const float e = __expf(-fabsf(g));                 // in (0, 1]: nothing overflows
    const float r = __fdividef(1.0f, 1.0f + e);
    return g * (g >= 0.f ? r : e * r) * u;
  }
  return g / (1.0f + expf(-g)) * u;
}

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total8, int paired) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total8) return;
  const unsigned per_row = (unsigned)inter >> 3;
  size_t n;
  int c;
  if (total8 <= 0xffffffffu) {                         // 32-bit division where it is enough
    n = (unsigned)i / per_row;
    c = (int)((unsigned)i % per_row) * 8;
  } else {
    n = i / per_row;
    c = (int)(i % per_row) * 8;
  }
  const T* row = gate_up + n * 2 * inter;
  const Vec8 g = load8(row + (paired ? 2 * c : c));
  const Vec8 u = load8(row + (paired ? 2 * c + 8 : inter + c));
  Vec8 y;
#pragma unroll
  for (int e = 0; e < 8; ++e) y.v[e] = silu_times<T>(g.v[e], u.v[e]);
  store8(out + n * inter + c, y);
}

}  // namespace ms
