// Paged grouped-query attention on the tensor cores (bfloat16 operands, float32 scores,
// softmax and accumulation), for prompt portions and decoded tokens alike.
//
// Work unit: one (request, key/value head, tile of query rows, split of the keys).  The
// query rows of a request and kv head are the pairs (token, query head of that kv head's
// group), token-major, so the G query heads that share a kv head sit in the same tile and
// every key/value tile read from the pool serves all of them.  A thread block has W warps
// of 16 rows each; key/value tiles of BN keys are gathered from the pages with 16-byte
// asynchronous copies into shared memory (double-buffered), then
//   S = Q K^T      mma.m16n8k16, K fragments by ldmatrix
//   online softmax (running maximum and sum per row, exp2 with the scale folded in)
//   O += P V       P re-used from the S accumulators as bf16, V fragments by ldmatrix.trans
// A key is visible to a row iff  pos - window < key <= pos  (pos: the row's token position).
// With one split the normalised result is written as bfloat16; with more, each split writes
// its normalised float32 partial result and log-sum-exp to scratch and a second kernel
// merges them.
#include "mma_common.cuh"
#include "attention_static.h"   // the declaration its users compile against is checked against the definition below

namespace ms {

// D head size, W warps, BN keys per tile, MT 16-row tiles per warp (a K/V fragment fetched from shared
// memory feeds MT MMAs), STAGES key/value tiles in shared memory (STAGES - 1 of them in flight while one
// is worked on).
template <int D, int W, int BN, int MT, int STAGES>
__global__ void __launch_bounds__(W * 32)
attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                     const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_tables, int table_stride,
                     const int* __restrict__ query_start, const int* __restrict__ context_lens, int page_size, int n_q,
                     int n_kv, float scale_log2, int window, __nv_bfloat16* __restrict__ out,
                     float* __restrict__ part_o, float* __restrict__ part_lse, int num_splits) {
  // The kernel before this one on the stream wrote the queries and the keys and values of this step's
  // tokens.  What the batch looks like (set up before the step's first kernel) and the keys and values of
  // earlier steps do not depend on it, so the first tiles of old keys are requested before the wait below.
  grid_dependency_launch();
  constexpr int BM = 16 * MT * W, THREADS = 32 * W, CHUNKS = D / 8;
  constexpr bool Q_IN_REGISTERS = MT == 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [BM][D]
  __nv_bfloat16* k_s = q_s + BM * D;                                        // [STAGES][BN][D]
  __nv_bfloat16* v_s = k_s + STAGES * BN * D;                               // [STAGES][BN][D]
  long long* row_offset = reinterpret_cast<long long*>(v_s + STAGES * BN * D);   // [STAGES][BN] pool offset of a key row, -1: none

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv_head = blockIdx.y;
  const int request = blockIdx.z / num_splits, split = blockIdx.z % num_splits;
  const int group = n_q / n_kv;
  const int q0 = query_start[request];
  const int q_len = query_start[request + 1] - q0;
  const int ctx = context_lens[request];
  const int rows_total = q_len * group;
  // Query tiles are taken from the end of the request: under the causal mask the last tiles have the
  // most keys, and starting them first keeps the tail of the launch short.
  const int row0 = ((rows_total + BM - 1) / BM - 1 - (int)blockIdx.x) * BM;
  if (row0 < 0) {
    grid_dependency_wait();
    return;
  }
  const int first_pos = ctx - q_len;                     // position of the request's first query token
  const int t_lo = row0 / group;
  const int last_row = min(rows_total, row0 + BM) - 1;
  const int t_hi = last_row / group;
  int key_begin = 0;
  if (window > 0) key_begin = max(0, first_pos + t_lo - window + 1);
  const int key_end = first_pos + t_hi + 1;
  const int tile_begin = (key_begin / BN) * BN;
  const int n_tiles = (key_end - tile_begin + BN - 1) / BN;
  const int tiles_per_split = (n_tiles + num_splits - 1) / num_splits;
  const int tile_lo = split * tiles_per_split;
  const int tile_hi = min(n_tiles, tile_lo + tiles_per_split);
  const int* table = block_tables + (size_t)request * table_stride;

  // rows of this thread in the mma layout: for each of the warp's MT tiles, rows (lane / 4) and (lane / 4) + 8
  const int quad_row = lane >> 2, quad_col = lane & 3;
  const int warp_row0 = row0 + warp * 16 * MT;
  auto thread_row = [&](int mt, int half) { return warp_row0 + mt * 16 + quad_row + half * 8; };

  if (tile_lo >= tile_hi) {                               // nothing to do for this split
    grid_dependency_wait();
    if (num_splits > 1 && quad_col == 0) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int row = thread_row(mt, half);
          if (row < rows_total) {
            const size_t index = ((size_t)(q0 + row / group) * n_q + kv_head * group + row % group);
            part_lse[index * num_splits + split] = -INFINITY;
          }
        }
    }
    return;
  }

  // Where each key row of a tile lies in the pool is looked up once per row (block table, page
  // arithmetic) and kept in shared memory; the copies then only add the chunk offset.  The offsets of
  // tile t + STAGES are computed while tile t is being worked on, into the buffer that tile t used.
  auto find_rows = [&](int tile, int buffer) {
    const int key0 = tile_begin + tile * BN;
    for (int r = tid; r < BN; r += THREADS) {
      const int key = key0 + r;
      long long offset = -1;
      if (tile < tile_hi && key < key_end) {
        const int page = table[key / page_size];
        offset = (((long long)page * n_kv + kv_head) * page_size + key % page_size) * D;
      }
      row_offset[buffer * BN + r] = offset;
    }
  };
  auto load_tile = [&](int stage) {
    __nv_bfloat16* ks = k_s + stage * BN * D;
    __nv_bfloat16* vs = v_s + stage * BN * D;
    const long long* offsets = row_offset + stage * BN;
#pragma unroll 4
    for (int i = tid; i < BN * CHUNKS; i += THREADS) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const long long offset = offsets[r];
      const bool valid = offset >= 0;
      const long long at = valid ? offset + c * 8 : 0;
      cp_async_16(tile_ptr<D>(ks, r, c), k_pool + at, valid);
      cp_async_16(tile_ptr<D>(vs, r, c), v_pool + at, valid);
    }
  };

#pragma unroll
  for (int s = 0; s < STAGES; ++s) find_rows(tile_lo + s, s);
  __syncthreads();
  // a tile that ends before the request's first new token holds keys of earlier steps only
  auto old_keys_only = [&](int s) { return tile_begin + (tile_lo + s + 1) * BN <= first_pos; };
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s)
    if (tile_lo + s < tile_hi && old_keys_only(s)) load_tile(s);
  cp_async_commit();
  grid_dependency_wait();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s)
    if (tile_lo + s < tile_hi && !old_keys_only(s)) load_tile(s);
  // ---- Q tile to shared memory
  for (int i = tid; i < BM * CHUNKS; i += THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const int row = row0 + r;
    const bool valid = row < rows_total;
    const __nv_bfloat16* src = q;
    if (valid) src = q + ((size_t)(q0 + row / group) * n_q + kv_head * group + row % group) * D + c * 8;
    cp_async_16(tile_ptr<D>(q_s, r, c), src, valid);
  }
  cp_async_commit();

  cp_async_wait<0>();            // Q and the first tiles have landed
  __syncthreads();

  unsigned q_frag[Q_IN_REGISTERS ? D / 16 : 1][4];
  auto q_fragment_address = [&](int mt, int kk) {
    const int r = (warp * MT + mt) * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = kk * 2 + (lane >> 4);
    return tile_ptr<D>(q_s, r, c);
  };
  if (Q_IN_REGISTERS) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) ldmatrix_x4(q_frag[kk], q_fragment_address(0, kk));
  }

  float acc_o[MT][D / 8][4];
  float m_run[MT][2], l_run[MT][2];
  int pos[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc_o[mt][n][e] = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      m_run[mt][half] = -INFINITY;
      l_run[mt][half] = 0.f;
      pos[mt][half] = first_pos + thread_row(mt, half) / group;
    }
  }

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int stage = (tile - tile_lo) % STAGES;
    if (tile + STAGES - 1 < tile_hi) load_tile((stage + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    find_rows(tile + STAGES, stage);     // this tile's copies have landed; its offsets are no longer needed
    const __nv_bfloat16* ks = k_s + stage * BN * D;
    const __nv_bfloat16* vs = v_s + stage * BN * D;
    const int key0 = tile_begin + tile * BN;

    // ---- S = Q K^T
    float acc_s[MT][BN / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < BN / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_s[mt][n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      unsigned a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (Q_IN_REGISTERS) {
#pragma unroll
          for (int e = 0; e < 4; ++e) a[mt][e] = q_frag[kk][e];
        } else {
          ldmatrix_x4(a[mt], q_fragment_address(mt, kk));
        }
      }
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        unsigned b[4];
        const int r = np * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(ks), r, c));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(acc_s[mt][2 * np], a[mt], b[0], b[1]);
          mma_bf16(acc_s[mt][2 * np + 1], a[mt], b[2], b[3]);
        }
      }
    }

    // ---- mask and online softmax (scores are scaled inside the exponent)
    const bool full = (key0 + BN - 1 <= first_pos + t_lo) && (window <= 0 || key0 >= first_pos + t_hi - window + 1);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (!full) {
            const int key = key0 + n * 8 + quad_col * 2 + (e & 1);
            const int p = pos[mt][e >> 1];
            const bool visible = key <= p && (window <= 0 || key > p - window);
            if (!visible) acc_s[mt][n][e] = -INFINITY;
          }
          tile_max[e >> 1] = fmaxf(tile_max[e >> 1], acc_s[mt][n][e]);
        }
      }
      float base[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float v = tile_max[half];
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
        const float updated = fmaxf(m_run[mt][half], v);
        base[half] = updated == -INFINITY ? 0.f : updated * scale_log2;
        corr[half] = exp2f(m_run[mt][half] * scale_log2 - base[half]);      // m == -inf gives 0
        m_run[mt][half] = updated;
      }
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc_s[mt][n][e] = exp2f(acc_s[mt][n][e] * scale_log2 - base[e >> 1]);
          sum[e >> 1] += acc_s[mt][n][e];
        }
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) l_run[mt][half] = l_run[mt][half] * corr[half] + sum[half];
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        acc_o[mt][n][0] *= corr[0];
        acc_o[mt][n][1] *= corr[0];
        acc_o[mt][n][2] *= corr[1];
        acc_o[mt][n][3] *= corr[1];
      }
    }

    // ---- O += P V
#pragma unroll
    for (int kp = 0; kp < BN / 16; ++kp) {
      unsigned p[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        p[mt][0] = pack_bf16(acc_s[mt][2 * kp][0], acc_s[mt][2 * kp][1]);
        p[mt][1] = pack_bf16(acc_s[mt][2 * kp][2], acc_s[mt][2 * kp][3]);
        p[mt][2] = pack_bf16(acc_s[mt][2 * kp + 1][0], acc_s[mt][2 * kp + 1][1]);
        p[mt][3] = pack_bf16(acc_s[mt][2 * kp + 1][2], acc_s[mt][2 * kp + 1][3]);
      }
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        unsigned b[4];
        const int r = kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = np * 2 + (lane >> 4);
        ldmatrix_x4_trans(b, tile_ptr<D>(const_cast<__nv_bfloat16*>(vs), r, c));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(acc_o[mt][2 * np], p[mt], b[0], b[1]);
          mma_bf16(acc_o[mt][2 * np + 1], p[mt], b[2], b[3]);
        }
      }
    }
    __syncthreads();       // all warps are done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- finish: row sums across the quad, normalise, store
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float l = l_run[mt][half];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const int row = thread_row(mt, half);
      if (row >= rows_total) continue;
      const float m = m_run[mt][half];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t index = (size_t)(q0 + row / group) * n_q + kv_head * group + row % group;
      if (num_splits == 1) {
        __nv_bfloat16* dst = out + index * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
          const unsigned packed = pack_bf16(acc_o[mt][n][2 * half] * inv, acc_o[mt][n][2 * half + 1] * inv);
          *reinterpret_cast<unsigned*>(dst + n * 8 + quad_col * 2) = packed;
        }
      } else {
        float* dst = part_o + (index * num_splits + split) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
          *reinterpret_cast<float2*>(dst + n * 8 + quad_col * 2) =
              make_float2(acc_o[mt][n][2 * half] * inv, acc_o[mt][n][2 * half + 1] * inv);
        if (quad_col == 0) part_lse[index * num_splits + split] = l > 0.f ? m * scale_log2 + log2f(l) : -INFINITY;
      }
    }
  }
}

// Thread blocks of the single-token variant that fit on the whole GPU at once (0 if it cannot be asked).
template <int D, int W, int BN, int MT, int STAGES>
int attention_block_slots() {
  static int slots = -1;
  if (slots < 0) {
    constexpr int BM = 16 * MT * W;
    const size_t smem = (size_t)(BM + 2 * STAGES * BN) * D * sizeof(__nv_bfloat16) + STAGES * BN * sizeof(long long);
    auto kernel = attention_mma_kernel<D, W, BN, MT, STAGES>;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, W * 32, smem) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    slots = sms * per_sm;
  }
  return slots;
}

template <int D, int W, int BN, int MT, int STAGES>
int launch_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                         int table_stride, const int* query_start, const int* context_lens, int page_size, int n_q,
                         int n_kv, float scale, int window, void* out, float* part_o, float* part_lse, int num_splits,
                         int n_requests, int max_query_len, int n_tokens, cudaStream_t stream) {
  constexpr int BM = 16 * MT * W;
  const size_t smem = (size_t)(BM + 2 * STAGES * BN) * D * sizeof(__nv_bfloat16) + STAGES * BN * sizeof(long long);
  auto kernel = attention_mma_kernel<D, W, BN, MT, STAGES>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("attention: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int group = n_q / n_kv;
  const long long tiles = ((long long)max_query_len * group + BM - 1) / BM;
  MS_REQUIRE(tiles <= 2147483647LL && (long long)n_requests * num_splits <= 65535 && n_kv <= 65535,
             "attention: grid %lld x %d x %lld exceeds the launch limits", tiles, n_kv, (long long)n_requests * num_splits);
  dim3 grid((unsigned)tiles, n_kv, n_requests * num_splits);
  const float scale_log2 = scale * 1.4426950408889634f;
  ms::launch(kernel, grid, W * 32, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                                         (const __nv_bfloat16*)v_pool, block_tables, table_stride, query_start,
                                         context_lens, page_size, n_q, n_kv, scale_log2, window, (__nv_bfloat16*)out,
                                         part_o, part_lse, num_splits);
  MS_CHECK_LAUNCH("attention_mma");
  if (num_splits > 1) {
    const int items = n_tokens * n_q;
    launch_attention_combine<D>(part_o, part_lse, (__nv_bfloat16*)out, num_splits, items, stream);
    MS_CHECK_LAUNCH("attention_combine");
  }
  return 0;
}

}  // namespace ms

using namespace ms;

// Head sizes this kernel is built for; other sizes use the general kernel.
MS_EXPORT int ms_attention_mma_supports(int head_dim) { return head_dim == 32 || head_dim == 64 || head_dim == 128; }

// In how many parts the keys of a step of single tokens should be split (1 for anything else).  A merge
// inside the attention kernel (the last split to finish merges, found by a ticket counter) was tried and
// was slower than the separate merge kernel: the memory fence every block then needs costs more.
MS_EXPORT int ms_attention_mma_splits(int d, int n_requests, int n_kv, int n_q, int max_query_len, int max_context_len) {
  if (n_kv <= 0 || (long long)max_query_len * (n_q / n_kv) > 16) return 1;
  int slots = 0;
  if (d == 128) slots = attention_block_slots<128, 1, 32, 1, 2>();
  else if (d == 64) slots = attention_block_slots<64, 1, 64, 1, 2>();
  else if (d == 32) slots = attention_block_slots<32, 1, 64, 1, 2>();
  const int base = n_requests * n_kv;
  if (slots <= 0 || base <= 0) return 1;
  // The blocks are one warp each, so what hides their latencies is how many of them are resident: pick the
  // smallest split count whose blocks fill whole waves to at least 90 % (each part keeping 64 keys or
  // more), else the count that fills them best.
  // a part keeps 64 keys (two tiles) or more: with one request the 64 parts of a 4,096-token context made the step 5.6 %
  // faster than 32 parts of 128 keys (a block's tiles are a chain of memory latencies), with two or more nothing changed
  int limit = max_context_len / 64;
  if (limit > 64) limit = 64;
  if (limit < 1) limit = 1;
  int splits = 1;
  double best = 0.0;
  for (int s = 1; s <= limit; ++s) {
    const long long blocks = (long long)base * s;
    const long long waves = (blocks + slots - 1) / slots;
    const double fill = (double)blocks / (double)(waves * slots);
    if (fill >= 0.9) {
      splits = s;
      break;
    }
    if (fill > best + 1e-9) {
      best = fill;
      splits = s;
    }
  }
  return splits < 1 ? 1 : splits;
}

// q, out [n_tokens, n_q, d] bfloat16; pools of one layer [pages, n_kv, page_size, d]; block_tables
// [n_requests, table_stride]; query_start [n_requests + 1]; context_lens [n_requests] (lengths after
// this step's tokens).  Request r's tokens query_start[r] .. query_start[r+1] are the last ones of its
// context.  num_splits > 1 needs part_o [n_tokens * n_q * num_splits * d] and part_lse
// [n_tokens * n_q * num_splits] float32 scratch and is meant for steps of single tokens.
MS_EXPORT int ms_paged_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                     int table_stride, const int* query_start, const int* context_lens,
                                     int page_size, int n_q, int n_kv, int d, float scale, int window, void* out,
                                     float* part_o, float* part_lse, int num_splits, int n_requests,
                                     int max_query_len, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || n_requests == 0) return 0;
  MS_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention: %d query heads are not a multiple of %d key/value heads", n_q, n_kv);
  MS_REQUIRE(page_size > 0 && max_query_len > 0, "attention: page size %d, longest portion %d", page_size, max_query_len);
  MS_REQUIRE(num_splits >= 1 && num_splits <= 64 && (num_splits == 1 || (part_o && part_lse)),
             "attention: %d splits (1..64) need scratch", num_splits);
  // Steps of single tokens: one warp per block (its 16 rows hold the group's query heads), two tiles in
  // shared memory (small blocks: more of them are resident).  Prompt portions: four warps of 32 rows each, two tiles.
  const bool small = (long long)max_query_len * (n_q / n_kv) <= 16;
#define MS_ATTENTION_CASE(D, W, BN, MT, STAGES)                                                                       \
  return launch_attention_mma<D, W, BN, MT, STAGES>(q, k_pool, v_pool, block_tables, table_stride, query_start,       \
                                                    context_lens, page_size, n_q, n_kv, scale, window, out, part_o,  \
                                                    part_lse, num_splits, n_requests, max_query_len, n_tokens, stream)
  if (d == 128) { if (small) { MS_ATTENTION_CASE(128, 1, 32, 1, 2); } else { MS_ATTENTION_CASE(128, 4, 64, 2, 2); } }
  if (d == 64) { if (small) { MS_ATTENTION_CASE(64, 1, 64, 1, 2); } else { MS_ATTENTION_CASE(64, 4, 64, 2, 2); } }
  if (d == 32) { if (small) { MS_ATTENTION_CASE(32, 1, 64, 1, 2); } else { MS_ATTENTION_CASE(32, 4, 64, 2, 2); } }
#undef MS_ATTENTION_CASE
  MS_FAIL("attention: the tensor-core kernel is not built for head size %d", d);
}

// ---------------------------------------------------------------------------------------------
// Split-key attention for callers that must not allocate (declared in attention_static.h).
//
// The split-key path above needs float32 scratch for the partial results of every split, which
// its caller allocates.  This entry point keeps that scratch in a fixed array inside the library
// instead, so a caller that cannot call cudaMalloc (a plug-in running inside another program's
// memory pool, a real-time loop that may not block in the allocator, a process whose device memory
// was handed out completely at start-up) can still run attention with its keys split.
namespace ms {
constexpr size_t kStaticScratchFloats = size_t(2) << 20;   // 8 MiB per GPU that loads the library
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
constexpr int kMaxDevices = 64;
static float* g_static_scratch_ptr[kMaxDevices] = {};
}  // namespace ms

MS_EXPORT int ms_paged_attention_decode_static(const void* q, const void* k_pool, const void* v_pool,
                                               const int* block_tables, int table_stride, const int* query_start,
                                               const int* context_lens, int page_size, int n_q, int n_kv, int d,
                                               float scale, int window, void* out, int num_splits, int n_requests,
                                               int n_tokens, cudaStream_t stream) {
  MS_REQUIRE(num_splits >= 1 && num_splits <= 64, "attention (static scratch): %d splits outside 1..64", num_splits);
  MS_REQUIRE(ms_attention_mma_supports(d), "attention (static scratch): head size %d is not built (32, 64, 128 are)", d);
  MS_REQUIRE(n_tokens == n_requests, "attention (static scratch): one token per request is expected (%d tokens, %d requests)",
             n_tokens, n_requests);
  const size_t rows = (size_t)n_tokens * (size_t)n_q * (size_t)num_splits;
  const size_t needed = rows * (size_t)(d + 1);
  MS_REQUIRE(needed <= kStaticScratchFloats,
             "attention (static scratch): tokens %d x heads %d x splits %d x (head size %d + 1) = %zu floats exceed the "
             "built-in scratch of %zu floats; use fewer splits or the entry point that takes scratch from its caller",
             n_tokens, n_q, num_splits, d, needed, (size_t)kStaticScratchFloats);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  MS_REQUIRE(e == cudaSuccess && device >= 0 && device < kMaxDevices, "attention (static scratch): no usable current device (%s)",
             cudaGetErrorString(e));
  if (g_static_scratch_ptr[device] == nullptr) {
    // First call on this device: ask the runtime where this device keeps its copy of the array.  In host
    // code the array's name is only a handle; passing it to a kernel would hand over a host address.
    float* address = nullptr;
    e = cudaGetSymbolAddress((void**)&address, g_static_scratch);
    MS_REQUIRE(e == cudaSuccess && address != nullptr, "attention (static scratch): cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
    g_static_scratch_ptr[device] = address;
  }
  float* part_o = g_static_scratch_ptr[device];
  float* part_lse = part_o + rows * (size_t)d;
  // Nothing in the scratch has to start at zero: every split of every row writes its log-sum-exp (minus
  // infinity when it had no keys), and a partial result is read only where that value is finite.
  return ms_paged_attention_mma(q, k_pool, v_pool, block_tables, table_stride, query_start, context_lens, page_size,
                                n_q, n_kv, d, scale, window, out, part_o, part_lse, num_splits, n_requests, 1, n_tokens,
                                stream);
}
