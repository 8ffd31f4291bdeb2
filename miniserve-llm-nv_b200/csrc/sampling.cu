// Next-token choice on the device from rows of float32 logits.
//
// A row without filters (argmax, or temperature alone) is an argmax over the vocabulary, of the logits or
// of the logits plus noise: a first kernel takes it in chunks, many thread blocks per row, and the second
// kernel merges the chunks' candidates.  A row with top-k or top-p goes through the second kernel alone,
// one thread block for the row.
//
// temperature == 0: argmax, the lowest index among equal maxima.
// otherwise, in this order: divide by the temperature; keep the top_k largest
// (top_k == 0: all; among equal values the lower index first); keep the nucleus
// (in descending order a token stays while the probability mass before it is at most
// top_p); draw from the softmax of what is left.  The draw is argmax(x_i + g_i) with
// Gumbel noise g_i = -log(-log(u_i)), u_i from Philox-4x32-10 keyed by the request's
// seed at counter (i / 4, draw index): it has the softmax as its distribution, needs no
// running sum, and depends on nothing but the request's own seed and draw index.
//
// The filters need no sort: a threshold on the (order-preserving) bit pattern of the
// values is found bit by bit with block-wide counts, then an index bound among the values
// equal to the threshold.  All block-wide sums run in a fixed order.
#include "common.cuh"

namespace ms {

constexpr int kSampleThreads = 1024;

struct SamplingRecord {  // one per state slot; 8 x 32 bit
  float temperature;
  float top_p;
  int top_k;
  unsigned seed_lo;
  unsigned seed_hi;
  int reserved[3];
};

__device__ __forceinline__ unsigned order_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void philox4x32_10(unsigned c0, unsigned c1, unsigned c2, unsigned c3, unsigned k0,
                                              unsigned k1, unsigned out[4]) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const unsigned hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const unsigned hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const unsigned n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float gumbel_from_word(unsigned w) {
  const float u = ((float)(w >> 8) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

struct ArgBest {
  float value;
  int index;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ ArgBest block_argmax(ArgBest v, ArgBest* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other;
    other.value = __shfl_xor_sync(0xffffffffu, v.value, o);
    other.index = __shfl_xor_sync(0xffffffffu, v.index, o);
    v = better(v, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  ArgBest total = scratch[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) total = better(total, scratch[w]);
  return total;
}

__device__ int block_count(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += scratch[w];
  return total;
}

// The kept set is { i : key_i > thr  or  (key_i == thr and i < bound) }.
struct Kept {
  unsigned thr;
  int bound;
  __device__ __forceinline__ bool has(unsigned key, int i) const { return key > thr || (key == thr && i < bound); }
};

// Largest b <= vocab with #{ i < b : key_i == thr } <= need.
__device__ int index_bound(const float* row, float temperature, int vocab, unsigned thr, int need, int* iscratch) {
  int b = 0;
  for (int bit = 30; bit >= 0; --bit) {
    const long long cand = (long long)b | (1LL << bit);
    if (cand > vocab) continue;
    int c = 0;
    for (int i = threadIdx.x; i < (int)cand; i += blockDim.x) c += order_key(row[i] / temperature) == thr;
    if (block_count(c, iscratch) <= need) b = (int)cand;
  }
  return b;
}

constexpr int kChunkThreads = 256;
constexpr int kChunk = 4096;                 // logits per block of the first kernel (a multiple of 4)

__device__ __forceinline__ bool without_filters(const SamplingRecord& rec, int vocab) {
  return rec.temperature == 0.f || ((rec.top_k <= 0 || rec.top_k >= vocab) && rec.top_p >= 1.0f);
}

// Block (chunk, row): the best of logits (or logits / temperature + noise) [chunk * kChunk, + kChunk) of a
// row without filters, to candidates[row * chunks + chunk].  The arithmetic is that of sample_kernel.
__global__ void __launch_bounds__(kChunkThreads)
sample_chunk_kernel(const float* __restrict__ logits, int row_stride, int vocab,
                    const SamplingRecord* __restrict__ records, const int* __restrict__ slot_of_row,
                    const int* __restrict__ draw_index, ArgBest* __restrict__ candidates) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ ArgBest ascratch[32];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  SamplingRecord rec;
  if (records) {
    rec = records[slot_of_row[r]];
  } else {
    rec.temperature = 0.f;
    rec.top_k = 0;
    rec.top_p = 1.f;
  }
  if (!without_filters(rec, vocab)) return;
  const bool greedy = rec.temperature == 0.f;
  const unsigned step = greedy ? 0u : (unsigned)draw_index[r];
  const bool vector_ok = (row_stride % 4 == 0) && (reinterpret_cast<uintptr_t>(logits) % 16 == 0);
  ArgBest best{-INFINITY, 0x7fffffff};
  const int first_group = chunk * (kChunk / 4), groups = (vocab + 3) / 4;
  for (int g = first_group + threadIdx.x; g < first_group + kChunk / 4 && g < groups; g += kChunkThreads) {
    float x[4];
    const int i0 = 4 * g;
    if (vector_ok && i0 + 4 <= vocab) {
      const float4 v = *reinterpret_cast<const float4*>(row + i0);
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = i0 + j < vocab ? row[i0 + j] : -INFINITY;
    }
    if (greedy) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (i0 + j < vocab && x[j] > best.value) best = ArgBest{x[j], i0 + j};
    } else {
      unsigned words[4];
      philox4x32_10((unsigned)g, step, 0u, 0u, rec.seed_lo, rec.seed_hi, words);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (i0 + j >= vocab) break;
        const float v = x[j] / rec.temperature + gumbel_from_word(words[j]);
        if (v > best.value) best = ArgBest{v, i0 + j};
      }
    }
  }
  best = block_argmax(best, ascratch);
  if (threadIdx.x == 0) candidates[(size_t)r * gridDim.x + chunk] = best;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int row_stride, int vocab, const SamplingRecord* __restrict__ records,
              const int* __restrict__ slot_of_row, const int* __restrict__ draw_index, int* __restrict__ out,
              const ArgBest* __restrict__ candidates, int chunks) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float fscratch[32];
  __shared__ int iscratch[32];
  __shared__ ArgBest ascratch[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  SamplingRecord rec;
  if (records) {
    rec = records[slot_of_row[r]];
  } else {
    rec.temperature = 0.f;
    rec.top_k = 0;
    rec.top_p = 1.f;
  }

  if (candidates != nullptr && without_filters(rec, vocab)) {      // the first kernel has been over this row
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) best = better(best, candidates[(size_t)r * chunks + c]);
    best = block_argmax(best, ascratch);
    if (threadIdx.x == 0) out[r] = best.index == 0x7fffffff ? 0 : best.index;
    return;
  }

  if (rec.temperature == 0.f) {
    ArgBest best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (v > best.value) best = ArgBest{v, i};
    }
    best = block_argmax(best, ascratch);
    if (threadIdx.x == 0) out[r] = best.index == 0x7fffffff ? 0 : best.index;
    return;
  }

  // x_i = logit_i / temperature, formed as in the plain rule (a float32 division).
  const float temperature = rec.temperature;
  auto scaled = [&](int i) { return row[i] / temperature; };
  Kept kept{0u, vocab};

  if (rec.top_k > 0 && rec.top_k < vocab) {
    const int k = rec.top_k;
    unsigned thr = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = thr | (1u << bit);
      int c = 0;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += order_key(scaled(i)) >= cand;
      if (block_count(c, iscratch) >= k) thr = cand;
    }
    int c_gt = 0, c_eq = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const unsigned key = order_key(scaled(i));
      c_gt += key > thr;
      c_eq += key == thr;
    }
    c_gt = block_count(c_gt, iscratch);
    c_eq = block_count(c_eq, iscratch);
    const int need = k - c_gt;
    kept.thr = thr;
    if (need < c_eq) kept.bound = index_bound(row, temperature, vocab, thr, need, iscratch);
  }

  if (rec.top_p < 1.0f) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, scaled(i));
    {
      ArgBest mb = block_argmax(ArgBest{m, 0}, ascratch);
      m = mb.value;
    }
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float x = scaled(i);
      if (kept.has(order_key(x), i)) z += expf(x - m);
    }
    z = block_sum(z, fscratch);
    const float limit = rec.top_p * z;
    // g(t) = [ mass of kept entries with key > t ] <= limit; find the smallest t with g(t).
    auto mass_above = [&](unsigned t) {
      float s = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = scaled(i);
        const unsigned key = order_key(x);
        if (key > t && kept.has(key, i)) s += expf(x - m);
      }
      return block_sum(s, fscratch);
    };
    unsigned s = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = s | (1u << bit);
      if (!(mass_above(cand) <= limit)) s = cand;
    }
    unsigned thr_p;
    if (mass_above(s) <= limit) thr_p = s; else thr_p = s + 1;   // s == 0xffffffff cannot fail: nothing lies above it
    if (thr_p >= kept.thr) {
      const float above = mass_above(thr_p);
      // value shared by the entries equal to the threshold, if any
      float tie_x = -INFINITY;
      int c_eq = 0;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = scaled(i);
        if (order_key(x) == thr_p && kept.has(thr_p, i)) {
          tie_x = x;
          ++c_eq;
        }
      }
      c_eq = block_count(c_eq, iscratch);
      tie_x = block_argmax(ArgBest{tie_x, 0}, ascratch).value;
      int bound = kept.thr == thr_p ? kept.bound : vocab;
      if (c_eq > 1) {
        const float each = expf(tie_x - m);
        const float room = (limit - above) / each;
        int n_keep = room >= (float)c_eq ? c_eq : (int)floorf(room) + 1;
        if (n_keep < 1) n_keep = 1;
        if (n_keep < c_eq) {
          const int b = index_bound(row, temperature, vocab, thr_p, n_keep, iscratch);
          if (b < bound) bound = b;
        }
      }
      kept.thr = thr_p;
      kept.bound = bound;
    }
  }

  const unsigned step = (unsigned)draw_index[r];
  ArgBest best{-INFINITY, 0x7fffffff};
  const int groups = (vocab + 3) / 4;
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    unsigned words[4];
    philox4x32_10((unsigned)g, step, 0u, 0u, rec.seed_lo, rec.seed_hi, words);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = 4 * g + j;
      if (i >= vocab) break;
      const float x = scaled(i);
      if (!kept.has(order_key(x), i)) continue;
      const float v = x + gumbel_from_word(words[j]);
      if (v > best.value) best = ArgBest{v, i};
    }
  }
  best = block_argmax(best, ascratch);
  if (threadIdx.x == 0) out[r] = best.index == 0x7fffffff ? 0 : best.index;
}

}  // namespace ms

using namespace ms;

// logits [n_rows, row_stride] float32, the first `vocab` entries of a row are used.
// records: [slots, 8] 32-bit words (temperature, top_p as float; top_k, seed low, seed high
// as integers; three unused), or null for argmax on every row.  slot_of_row, draw_index [n_rows].
// scratch: room for n_rows * ms_sample_chunks(vocab) pairs of 32-bit words (contents arbitrary), or null,
// in which case every row is handled by one thread block.
MS_EXPORT int ms_sample_chunks(int vocab) { return (vocab + kChunk - 1) / kChunk; }

MS_EXPORT int ms_sample(const float* logits, int row_stride, int vocab, const void* records, const int* slot_of_row,
                        const int* draw_index, int* out, int n_rows, void* scratch, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  MS_REQUIRE(vocab > 0 && row_stride >= vocab, "sample: vocabulary %d, row stride %d", vocab, row_stride);
  MS_REQUIRE(records == nullptr || (slot_of_row != nullptr && draw_index != nullptr),
             "sample: sampling records need slot and draw index arrays");
  const int chunks = ms_sample_chunks(vocab);
  if (scratch != nullptr) {
    MS_REQUIRE(n_rows <= 65535, "sample: %d rows in one call is too many", n_rows);
    ms::launch(sample_chunk_kernel, dim3(chunks, n_rows), dim3(kChunkThreads), 0, stream, logits, row_stride, vocab,
               (const SamplingRecord*)records, slot_of_row, draw_index, (ArgBest*)scratch);
    MS_CHECK_LAUNCH("sample (chunks)");
  }
  ms::launch(sample_kernel, n_rows, kSampleThreads, 0, stream, logits, row_stride, vocab, (const SamplingRecord*)records,
             slot_of_row, draw_index, out, (const ArgBest*)scratch, chunks);
  MS_CHECK_LAUNCH("sample");
  return 0;
}
