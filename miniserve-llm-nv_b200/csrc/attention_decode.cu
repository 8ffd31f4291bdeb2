// Everything between the q/k/v projection and the split-key attention of a decode step in the attention kernel
// itself: per-head RMSNorm of q and k, rotation, and the append of k and v to the paged cache.
//
// As a kernel of its own, norm + rotation + append is one more link in the chain of dependent launches that a
// decode step is (2 to 3 us for a few KB of work).  Here:
//   - a thread block of one warp handles one (request, key/value head, split of the keys), as in
//     attention_mma.cu, and the splits' partial results are merged by the same second kernel;
//   - every key and value tile of the step is requested BEFORE the kernel waits for its predecessor: the
//     only key the step adds is the new token's own, and that one does not come from the cache.  The block
//     that owns the last split computes it (norm, rotation) from the projection's output after the wait,
//     stores it and the value to the cache for later steps, and puts both into its shared-memory tile in
//     place of whatever the cache held there;
//   - every block norms and rotates the group's query heads itself (two heads of 128 numbers here: less
//     work than reading them back from memory would be) straight into the shared-memory tile that feeds
//     the MMAs.
// Arithmetic as in the separate kernels: float32 norm and rotation rounded once to bfloat16, float32 scores
// and softmax, P rounded to bfloat16 for PV.
#include "mma_common.cuh"


namespace ms {
namespace fused {

constexpr int MAX_SPLITS = 64;     // what the merge kernel takes
constexpr int ROWS = 16;           // query rows of a block's MMA tile: the group's heads, the rest zeros

// elements of one half of a head per lane (the lane also holds their partners in the other half)
template <int D> __host__ __device__ constexpr int per_lane() { return D / 64; }

// Norm (optional) and half-split rotation (optional) of one head of D numbers spread over the warp: lane l
// holds elements l * E .. l * E + E - 1 in lo[] and the same of the second half in hi[].
template <int D>
__device__ __forceinline__ void norm_and_rotate(float (&lo)[per_lane<D>()], float (&hi)[per_lane<D>()], const void* weight,
                                                int weight_dtype, float eps, const float* cos_sin_row, int lane) {
  constexpr int E = per_lane<D>();
  if (weight != nullptr) {
    float squares = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) squares += lo[e] * lo[e] + hi[e] * hi[e];
    squares = warp_sum(squares);
    const float inv = 1.0f / sqrtf(squares / (float)D + eps);
#pragma unroll
    for (int e = 0; e < E; ++e) {
      lo[e] = lo[e] * inv * load_as_float(weight, weight_dtype, lane * E + e);
      hi[e] = hi[e] * inv * load_as_float(weight, weight_dtype, D / 2 + lane * E + e);
    }
  }
  if (cos_sin_row != nullptr) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float2 cs = *reinterpret_cast<const float2*>(cos_sin_row + 2 * (lane * E + e));
      const float a = lo[e], b = hi[e];
      lo[e] = a * cs.x - b * cs.y;
      hi[e] = b * cs.x + a * cs.y;
    }
  }
}

template <int D>
__device__ __forceinline__ void load_head(const __nv_bfloat16* src, float (&lo)[per_lane<D>()], float (&hi)[per_lane<D>()], int lane) {
  constexpr int E = per_lane<D>();
#pragma unroll
  for (int e = 0; e < E; ++e) {
    lo[e] = __bfloat162float(src[lane * E + e]);
    hi[e] = __bfloat162float(src[D / 2 + lane * E + e]);
  }
}

// Row `row` of a swizzled [rows][D] tile (or of a plain row in global memory: tile == false) receives the head.
template <int D, bool TILE>
__device__ __forceinline__ void store_head(__nv_bfloat16* base, int row, const float (&lo)[per_lane<D>()],
                                           const float (&hi)[per_lane<D>()], int lane) {
  constexpr int E = per_lane<D>();
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int c_lo = lane * E + e, c_hi = D / 2 + c_lo;
    __nv_bfloat16* at_lo = TILE ? tile_ptr<D>(base, row, c_lo >> 3) + (c_lo & 7) : base + c_lo;
    __nv_bfloat16* at_hi = TILE ? tile_ptr<D>(base, row, c_hi >> 3) + (c_hi & 7) : base + c_hi;
    *at_lo = __float2bfloat16_rn(lo[e]);
    *at_hi = __float2bfloat16_rn(hi[e]);
  }
}

template <int D, int BN, int STAGES>
__global__ void __launch_bounds__(32)
attention_decode_fused_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ slots,
                              const void* __restrict__ q_weight, const void* __restrict__ k_weight, int weight_dtype,
                              float eps, const float* __restrict__ cos_sin, __nv_bfloat16* __restrict__ k_pool,
                              __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ block_tables, int table_stride,
                              const int* __restrict__ query_start, const int* __restrict__ context_lens, int page_size,
                              int n_q, int n_kv, float scale_log2, int window, __nv_bfloat16* __restrict__ out,
                              float* __restrict__ part_o, float* __restrict__ part_lse, int num_splits) {
  grid_dependency_launch();
  constexpr int CHUNKS = D / 8, E = per_lane<D>();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [ROWS][D]
  __nv_bfloat16* k_s = q_s + ROWS * D;                                             // [STAGES][BN][D]
  __nv_bfloat16* v_s = k_s + STAGES * BN * D;                                      // [STAGES][BN][D]
  long long* row_offset = reinterpret_cast<long long*>(v_s + STAGES * BN * D);     // [STAGES][BN]; -1: no such key

  const int lane = threadIdx.x;
  const int kv_head = blockIdx.y;
  const int request = blockIdx.z / num_splits, split = blockIdx.z % num_splits;
  const int group = n_q / n_kv, heads = n_q + 2 * n_kv;
  const int token = query_start[request];
  const int ctx = context_lens[request];
  const int pos = ctx - 1;                                  // the new token's position: its own key is the last one
  const int slot = slots[token];
  const bool inject = slot >= 0;                            // else the key is in the cache already (another run wrote it this step)
  int key_begin = 0;
  if (window > 0) key_begin = max(0, pos - window + 1);
  const int key_end = ctx;
  const int tile_begin = (key_begin / BN) * BN;
  const int n_tiles = (key_end - tile_begin + BN - 1) / BN;
  const int tiles_per_split = (n_tiles + num_splits - 1) / num_splits;
  const int tile_lo = split * tiles_per_split;
  const int tile_hi = min(n_tiles, tile_lo + tiles_per_split);
  const bool has_keys = tile_lo < tile_hi;
  const bool owns_new_key = has_keys && tile_hi == n_tiles;
  const int* table = block_tables + (size_t)request * table_stride;
  const int quad_row = lane >> 2, quad_col = lane & 3;

  auto find_rows = [&](int tile, int buffer) {
    const int key0 = tile_begin + tile * BN;
    for (int r = lane; r < BN; r += 32) {
      const int key = key0 + r;
      long long offset = -1;
      if (tile < tile_hi && key < key_end && !(inject && key == pos)) {
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
    for (int i = lane; i < BN * CHUNKS; i += 32) {
      const int r = i / CHUNKS, c = i % CHUNKS;
      const long long offset = offsets[r];
      const bool valid = offset >= 0;
      const long long at = valid ? offset + c * 8 : 0;
      cp_async_16(tile_ptr<D>(ks, r, c), k_pool + at, valid);
      cp_async_16(tile_ptr<D>(vs, r, c), v_pool + at, valid);
    }
  };
  // a tile may be requested before the wait if nothing in it is written during this step
  auto settled = [&](int s) { return inject || tile_begin + (tile_lo + s + 1) * BN <= pos; };

  if (has_keys) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) find_rows(tile_lo + s, s);
    __syncwarp();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
      if (tile_lo + s < tile_hi && settled(s)) load_tile(s);
  }
  cp_async_commit();
  // zeros for the rows of the query tile that hold no head
  for (int i = lane; i < ROWS * CHUNKS; i += 32) *reinterpret_cast<uint4*>(q_s + i * 8) = make_uint4(0u, 0u, 0u, 0u);
  grid_dependency_wait();

  if (has_keys) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
      if (tile_lo + s < tile_hi && !settled(s)) load_tile(s);
  }
  cp_async_commit();
  __syncwarp();

  // ---- the group's query heads: norm, rotation, into the tile
  const __nv_bfloat16* token_row = qkv + (size_t)token * heads * D;
  const float* cos_sin_row = cos_sin != nullptr ? cos_sin + (size_t)token * D : nullptr;
  if (has_keys) {
    for (int h = 0; h < group; ++h) {
      float lo[E], hi[E];
      load_head<D>(token_row + (size_t)(kv_head * group + h) * D, lo, hi, lane);
      norm_and_rotate<D>(lo, hi, q_weight, weight_dtype, eps, cos_sin_row, lane);
      store_head<D, true>(q_s, h, lo, hi, lane);
    }
  }
  // ---- the new token's key and value: to the cache, and kept for this block's own last tile
  float k_lo[E], k_hi[E], v_lo[E], v_hi[E];
  if (owns_new_key && inject) {
    load_head<D>(token_row + (size_t)(n_q + kv_head) * D, k_lo, k_hi, lane);
    norm_and_rotate<D>(k_lo, k_hi, k_weight, weight_dtype, eps, cos_sin_row, lane);
    load_head<D>(token_row + (size_t)(n_q + n_kv + kv_head) * D, v_lo, v_hi, lane);
    const size_t at = (((size_t)(slot / page_size) * n_kv + kv_head) * page_size + slot % page_size) * D;
    store_head<D, false>(k_pool + at, 0, k_lo, k_hi, lane);
    store_head<D, false>(v_pool + at, 0, v_lo, v_hi, lane);
  }
  __syncwarp();

  float acc_o[D / 8][4];
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc_o[n][e] = 0.f;

  if (has_keys) {
    unsigned q_frag[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      ldmatrix_x4(q_frag[kk], tile_ptr<D>(q_s, (lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4)));

    for (int tile = tile_lo; tile < tile_hi; ++tile) {
      const int stage = (tile - tile_lo) % STAGES;
      if (tile + STAGES - 1 < tile_hi) load_tile((stage + STAGES - 1) % STAGES);
      cp_async_commit();
      cp_async_wait<STAGES - 1>();
      __syncwarp();
      find_rows(tile + STAGES, stage);     // this tile's copies have landed; its offsets are no longer needed
      __nv_bfloat16* ks = k_s + stage * BN * D;
      __nv_bfloat16* vs = v_s + stage * BN * D;
      const int key0 = tile_begin + tile * BN;
      if (inject && owns_new_key && tile == tile_hi - 1) {        // the new token's own key and value, not from the cache
        store_head<D, true>(ks, pos - key0, k_lo, k_hi, lane);
        store_head<D, true>(vs, pos - key0, v_lo, v_hi, lane);
        __syncwarp();
      }

      // ---- S = Q K^T
      float acc_s[BN / 8][4];
#pragma unroll
      for (int n = 0; n < BN / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_s[n][e] = 0.f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          unsigned b[4];
          const int r = np * 16 + (lane & 7) + (lane >> 4) * 8;
          const int c = kk * 2 + ((lane >> 3) & 1);
          ldmatrix_x4(b, tile_ptr<D>(ks, r, c));
          mma_bf16(acc_s[2 * np], q_frag[kk], b[0], b[1]);
          mma_bf16(acc_s[2 * np + 1], q_frag[kk], b[2], b[3]);
        }
      }

      // ---- mask and online softmax (scores are scaled inside the exponent); every row is the same token
      const bool full = key0 + BN - 1 <= pos && (window <= 0 || key0 >= pos - window + 1);
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (!full) {
            const int key = key0 + n * 8 + quad_col * 2 + (e & 1);
            const bool visible = key <= pos && (window <= 0 || key > pos - window);
            if (!visible) acc_s[n][e] = -INFINITY;
          }
          tile_max[e >> 1] = fmaxf(tile_max[e >> 1], acc_s[n][e]);
        }
      }
      float base[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float v = tile_max[half];
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
        const float updated = fmaxf(m_run[half], v);
        base[half] = updated == -INFINITY ? 0.f : updated * scale_log2;
        corr[half] = exp2f(m_run[half] * scale_log2 - base[half]);      // m == -inf gives 0
        m_run[half] = updated;
      }
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc_s[n][e] = exp2f(acc_s[n][e] * scale_log2 - base[e >> 1]);
          sum[e >> 1] += acc_s[n][e];
        }
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) l_run[half] = l_run[half] * corr[half] + sum[half];
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        acc_o[n][0] *= corr[0];
        acc_o[n][1] *= corr[0];
        acc_o[n][2] *= corr[1];
        acc_o[n][3] *= corr[1];
      }

      // ---- O += P V
#pragma unroll
      for (int kp = 0; kp < BN / 16; ++kp) {
        unsigned p[4];
        p[0] = pack_bf16(acc_s[2 * kp][0], acc_s[2 * kp][1]);
        p[1] = pack_bf16(acc_s[2 * kp][2], acc_s[2 * kp][3]);
        p[2] = pack_bf16(acc_s[2 * kp + 1][0], acc_s[2 * kp + 1][1]);
        p[3] = pack_bf16(acc_s[2 * kp + 1][2], acc_s[2 * kp + 1][3]);
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
          unsigned b[4];
          const int r = kp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = np * 2 + (lane >> 4);
          ldmatrix_x4_trans(b, tile_ptr<D>(vs, r, c));
          mma_bf16(acc_o[2 * np], p, b[0], b[1]);
          mma_bf16(acc_o[2 * np + 1], p, b[2], b[3]);
        }
      }
      __syncwarp();       // the warp is done with this stage before it is refilled
    }
  }
  cp_async_wait<0>();
  __syncwarp();

  // ---- finish: row sums across the quad, then store (one split) or leave the partial result for the merge kernel
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    float l = l_run[half];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = quad_row + half * 8;
    if (row >= group) continue;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const size_t index = (size_t)token * n_q + kv_head * group + row;
    if (num_splits == 1) {
      __nv_bfloat16* dst = out + index * D;
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        *reinterpret_cast<unsigned*>(dst + n * 8 + quad_col * 2) = pack_bf16(acc_o[n][2 * half] * inv, acc_o[n][2 * half + 1] * inv);
    } else {
      float* dst = part_o + (index * num_splits + split) * D;
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + quad_col * 2) = make_float2(acc_o[n][2 * half] * inv, acc_o[n][2 * half + 1] * inv);
      if (quad_col == 0) part_lse[index * num_splits + split] = l > 0.f ? m_run[half] * scale_log2 + log2f(l) : -INFINITY;
    }
  }
}

template <int D, int BN, int STAGES>
size_t shared_bytes() {
  return (size_t)(ROWS + 2 * STAGES * BN) * D * sizeof(__nv_bfloat16) + STAGES * BN * sizeof(long long);
}

template <int D, int BN, int STAGES>
int launch(const void* qkv, const int* slots, const void* q_weight, const void* k_weight, int weight_dtype, float eps,
           const float* cos_sin, void* k_pool, void* v_pool, const int* block_tables, int table_stride,
           const int* query_start, const int* context_lens, int page_size, int n_q, int n_kv, float scale, int window,
           void* out, float* part_o, float* part_lse, int num_splits, int n_requests, cudaStream_t stream) {
  auto kernel = attention_decode_fused_kernel<D, BN, STAGES>;
  const size_t smem = shared_bytes<D, BN, STAGES>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  MS_REQUIRE((long long)n_requests * num_splits <= 65535 && n_kv <= 65535, "attention_decode: grid %d x %lld exceeds the launch limits",
             n_kv, (long long)n_requests * num_splits);
  cudaError_t e = ms::launch(kernel, dim3(1, n_kv, n_requests * num_splits), dim3(32), smem, stream, (const __nv_bfloat16*)qkv, slots,
                             q_weight, k_weight, weight_dtype, eps, cos_sin, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                             block_tables, table_stride, query_start, context_lens, page_size, n_q, n_kv,
                             scale * 1.4426950408889634f, window, (__nv_bfloat16*)out, part_o, part_lse, num_splits);
  if (e != cudaSuccess) MS_FAIL("attention_decode: launch failed: %s", cudaGetErrorString(e));
  if (num_splits > 1) {
    const int items = n_requests * n_q;
    launch_attention_combine<D>(part_o, part_lse, (__nv_bfloat16*)out, num_splits, items, stream);
    MS_CHECK_LAUNCH("attention_combine");
  }
  return 0;
}

// Blocks of the kernel that the whole GPU holds at once (0: cannot be asked).
template <int D, int BN, int STAGES>
int block_slots() {
  static int slots = -1;
  if (slots < 0) {
    auto kernel = attention_decode_fused_kernel<D, BN, STAGES>;
    const size_t smem = shared_bytes<D, BN, STAGES>();
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 32, smem) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    slots = sms * per_sm;
  }
  return slots;
}

}  // namespace fused
}  // namespace ms

using namespace ms;

// Whether the fused kernel takes a decode step of these sizes: head size 64 or 128, at most 16 query heads per
// key/value head (they are the rows of one MMA tile).
MS_EXPORT int ms_attention_decode_fused_supports(int head_dim, int n_q, int n_kv) {
  if (n_kv <= 0 || n_q % n_kv != 0) return 0;
  return (head_dim == 64 || head_dim == 128) && n_q / n_kv <= fused::ROWS;
}

// In how many parts (1..64) the keys of every request should be split: the smallest count whose blocks fill whole
// waves of the GPU's block slots to at least 90 % (each part keeping 64 keys or more), else the count that fills
// them best.  The count depends on the batch's shape only (requests, longest context allowed), not on its content.
MS_EXPORT int ms_attention_decode_fused_splits(int head_dim, int n_requests, int n_kv, int max_context_len) {
  const int slots = head_dim == 128 ? fused::block_slots<128, 32, 2>() : fused::block_slots<64, 64, 2>();
  const long long base = (long long)n_requests * n_kv;
  if (slots <= 0 || base <= 0) return 1;
  // a part keeps 64 keys (two tiles) or more: with one request the 64 parts of a 4,096-token context made the step 5.6 %
  // faster than 32 parts of 128 keys (a block's tiles are a chain of memory latencies), with two or more nothing changed
  int limit = max_context_len / 64;
  if (limit > fused::MAX_SPLITS) limit = fused::MAX_SPLITS;
  if (limit < 1) limit = 1;
  int splits = 1;
  double best = 0.0;
  for (int s = 1; s <= limit; ++s) {
    const long long blocks = base * s, waves = (blocks + slots - 1) / slots;
    const double fill = (double)blocks / (double)(waves * slots);
    if (fill >= 0.9) return s;
    if (fill > best + 1e-9) {
      best = fill;
      splits = s;
    }
  }
  return splits;
}

// A decode step's attention from the fused projection's output to the attended heads, for requests of ONE new
// token each (query_start[r + 1] - query_start[r] == 1).
//   qkv [n_tokens, (n_q + 2 n_kv) * d] bfloat16: the projection's output, untouched;
//   slots [n_tokens]: page * page_size + offset where the token's key and value go (negative: the cache holds
//   them already and nothing is written); q_weight, k_weight [d] (float32: weight_dtype 0, bfloat16: 1) or null: no
//   norm; cos_sin [n_tokens, d / 2, 2] float32 or null: no rotation (half-split pairs over the whole head);
//   pools of one layer [pages, n_kv, page_size, d]; block_tables [n_requests, table_stride]; context_lens
//   [n_requests]: lengths including the new token; out [n_tokens, n_q, d] bfloat16; num_splits 1..64, and for more
//   than one split part_o [n_tokens * n_q * num_splits * d] and part_lse [n_tokens * n_q * num_splits] float32.
MS_EXPORT int ms_attention_decode_fused(const void* qkv, const int* slots, const void* q_weight, const void* k_weight,
                                        int weight_dtype, float eps, const float* cos_sin, void* k_pool, void* v_pool,
                                        const int* block_tables, int table_stride, const int* query_start,
                                        const int* context_lens, int page_size, int n_q, int n_kv, int d, float scale,
                                        int window, void* out, float* part_o, float* part_lse, int num_splits,
                                        int n_requests, cudaStream_t stream) {
  if (n_requests == 0) return 0;
  MS_REQUIRE(ms_attention_decode_fused_supports(d, n_q, n_kv), "attention_decode: head size %d with %d/%d heads is not taken", d, n_q, n_kv);
  MS_REQUIRE(num_splits >= 1 && num_splits <= fused::MAX_SPLITS && (num_splits == 1 || (part_o && part_lse)),
             "attention_decode: %d splits (1..%d) need scratch", num_splits, fused::MAX_SPLITS);
  MS_REQUIRE(page_size > 0, "attention_decode: page size %d", page_size);
  if (d == 128)
    return fused::launch<128, 32, 2>(qkv, slots, q_weight, k_weight, weight_dtype, eps, cos_sin, k_pool, v_pool, block_tables,
                                     table_stride, query_start, context_lens, page_size, n_q, n_kv, scale, window, out, part_o,
                                     part_lse, num_splits, n_requests, stream);
  return fused::launch<64, 64, 2>(qkv, slots, q_weight, k_weight, weight_dtype, eps, cos_sin, k_pool, v_pool, block_tables,
                                  table_stride, query_start, context_lens, page_size, n_q, n_kv, scale, window, out, part_o, part_lse,
                                  num_splits, n_requests, stream);
}
