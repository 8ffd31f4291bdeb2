// Paged grouped-query attention for prompt portions on the fifth-generation tensor cores.
//
// One thread block handles 128 query rows of one (request, key/value head): the rows are the pairs
// (token, query head of the kv head's group), token-major, so all heads of the group share each key and
// value tile.  Keys are walked in tiles of 128:
//   warp 0      one thread issues TMA loads: the query rows once (a 3-d box over tokens x heads x head
//               size), then per tile one box per cache page for K and for V, looked up in the request's
//               block table, into a ring of three or four tiles in shared memory (128-byte swizzle);
//   warp 1      one thread issues tcgen05.mma:  S = Q K^T  into one of two score buffers in tensor memory
//               (issued one tile ahead, so it overlaps the softmax of the tile before), and  PV = P V  with
//               P read from tensor memory and V as an MN-major operand from shared memory;
//   warps 2..9  two threads per query row, one for each half of a tile's keys (a warp reaches only its own
//               quarter of the tensor-memory lanes, so warps 2..5 take the first half and warps 6..9, which
//               own the same quarters, the second): read the row of S from tensor memory, mask by absolute
//               position, agree on the row maximum through shared memory, keep a running sum each
//               (float32, exp2 with the scale folded in) and write P as bfloat16 back into tensor memory
//               over the scores it came from.  The softmax sets the pace of the kernel (the MMAs of the
//               next tile run beside it), so halving a thread's share shortens every tile.  The output accumulates in
//               tensor memory across the tiles; it is rescaled only when a row's maximum has grown by more
//               than 2^8 since the last rescale (the exponent then stays small enough for bfloat16 and
//               float32, and the final division by the row sum makes the result exact all the same).
// Tensor memory: columns 0..255 two score buffers, 256..256+D the output.  All mbarrier waits are
// bounded; a wait that runs out sets the error flag and every role drains and returns.
#include "tcgen05.cuh"

namespace ms {
namespace t5a {

using namespace ms::t5;

constexpr int ROWS = 128, BN = 128, THREADS = 320, TMEM_COLUMNS = 512;
constexpr int HALF = BN / 2;               // keys of a tile per softmax thread
// key/value tiles in shared memory: three for head size 128 (32 KB of queries + 3 x 64 KB), four for 64
template <int D> constexpr int kv_stages() { return D == 128 ? 3 : 4; }

// 2^x by the special-function unit (ex2.approx): relative error about 2^-22, -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct Layout {
  static constexpr int KV_STAGES = kv_stages<D>();
  static constexpr int DBLOCKS = D / 64;                 // 128-byte column blocks of a row
  static constexpr int Q_BYTES = ROWS * D * 2;
  static constexpr int TILE_BYTES = BN * D * 2;          // one K or V tile
  static constexpr size_t TOTAL = (size_t)Q_BYTES + (size_t)KV_STAGES * 2 * TILE_BYTES + 1024;
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_tables,
                         int table_stride, const int* __restrict__ query_start, const int* __restrict__ context_lens,
                         int page_size, int n_q, int n_kv, float scale_log2, int window,
                         __nv_bfloat16* __restrict__ out, int* __restrict__ error_flag) {
  using L = Layout<D>;
  constexpr int KV_STAGES = L::KV_STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  auto k_stage = [&](int s) { return smem + L::Q_BYTES + (size_t)s * 2 * L::TILE_BYTES; };
  auto v_stage = [&](int s) { return k_stage(s) + L::TILE_BYTES; };
  __shared__ uint64_t q_full, k_full[KV_STAGES], v_full[KV_STAGES], kv_empty[KV_STAGES];
  // pv_done[j & 1]: the output is complete up to key tile j.  (A wait by parity only tells the completion that comes
  // next from the one before it: whoever waits for tile j's must know that the same barrier's last but one, tile
  // j - 2's, has happened.  The scores of tile j are multiplied behind the output of tile j - 2, so having seen them
  // is enough for tiles j - 1 and j; at the end the outputs are waited for in their order.)
  __shared__ uint64_t s_full[2], p_full[2], pv_done[2];
  __shared__ unsigned tmem_base_s;
  // [tile parity][half][row]: the two threads of a row agree on its maximum.  Shared memory is full to the
  // last kilobyte, so the maxima are exchanged as bfloat16, rounded up (any bound above the true maximum
  // serves: sums and output stay relative to the same value), and the same bytes carry the two row sums
  // at the end.
  __shared__ __align__(16) __nv_bfloat16 half_max_s[2][2][ROWS];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Blocks are handed out in the order of blockIdx.x, then y: with the kv head in x and the query tile in y
  // (last tiles, which have the most keys, first) the longest blocks of all heads start first, and the short
  // ones fill the gaps at the end.
  const int kv_head = blockIdx.x, request = blockIdx.z;
  const int group = n_q / n_kv;
  const int q0 = query_start[request];
  const int q_len = query_start[request + 1] - q0;
  const int ctx = context_lens[request];
  const int rows_total = q_len * group;
  const int row0 = ((rows_total + ROWS - 1) / ROWS - 1 - (int)blockIdx.y) * ROWS;   // last tiles first
  const bool active = row0 >= 0;
  const int first_pos = ctx - q_len;
  const int t_lo = active ? row0 / group : 0;
  const int t_hi = active ? (min(rows_total, row0 + ROWS) - 1) / group : 0;
  int key_begin = 0;
  if (window > 0) key_begin = max(0, first_pos + t_lo - window + 1);
  const int key_end = first_pos + t_hi + 1;
  const int tile_begin = (key_begin / BN) * BN;
  const int n_tiles = active ? (key_end - tile_begin + BN - 1) / BN : 0;
  const int* table = block_tables + (size_t)request * table_stride;

  if (warp == 0 && lane == 0) {
    mbar_init(&q_full, 1);
#pragma unroll
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 2 * ROWS);
    }
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLUMNS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const unsigned tmem_base = tmem_base_s;
  auto s_column = [&](int b) { return (unsigned)(b * BN); };
  const unsigned o_column = 2 * BN;

  grid_dependency_wait();
  grid_dependency_launch();

  if (active) {
    if (warp == 0) {
      // ---------------- producer: lane 0 announces the bytes, all lanes issue the page loads
      if (lane == 0) {
        mbar_expect_tx(&q_full, L::Q_BYTES);
#pragma unroll
        for (int db = 0; db < L::DBLOCKS; ++db)
          tma_load_3d(q_s + db * (ROWS * 128), &map_q, &q_full, db * 64, kv_head * group, q0 + t_lo);
      }
      const int pages_per_tile = BN / page_size;
      const int loads_per_tile = pages_per_tile * L::DBLOCKS;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % KV_STAGES;
        const unsigned phase = (j / KV_STAGES) & 1;
        if (lane == 0) {
          ok = mbar_wait(&kv_empty[stage], phase ^ 1, error_flag, 11);
          if (ok) {
            mbar_expect_tx(&k_full[stage], L::TILE_BYTES);
            mbar_expect_tx(&v_full[stage], L::TILE_BYTES);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const int key0 = tile_begin + j * BN;
        for (int i = lane; i < loads_per_tile; i += 32) {
          const int p = i / L::DBLOCKS, db = i % L::DBLOCKS;
          const int key = key0 + p * page_size;
          // pages past the context are replaced by the request's first page: finite numbers that the mask removes
          const int page = key < key_end ? table[key / page_size] : table[0];
          const int pool_row = (page * n_kv + kv_head) * page_size;
          const size_t at = (size_t)db * (BN * 128) + (size_t)(p * page_size) * 128;
          tma_load_2d(k_stage(stage) + at, &map_k, &k_full[stage], db * 64, pool_row);
          tma_load_2d(v_stage(stage) + at, &map_v, &v_full[stage], db * 64, pool_row);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        // ---------------- MMA issue
        constexpr unsigned idesc_s = umma_idesc(ROWS, BN, false);
        constexpr unsigned idesc_pv = umma_idesc(ROWS, D, true);
        auto issue_scores = [&](int j) {
          const int stage = j % KV_STAGES, b = j & 1;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t a_desc = umma_desc(q_s + (kk / 4) * (ROWS * 128)) + 2 * (kk % 4);
            const uint64_t b_desc = umma_desc(k_stage(stage) + (kk / 4) * (BN * 128)) + 2 * (kk % 4);
            umma_bf16(tmem_base + s_column(b), a_desc, b_desc, idesc_s, kk != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[b]);
        };
        bool ok = mbar_wait(&q_full, 0, error_flag, 12) && mbar_wait(&k_full[0], 0, error_flag, 13);
        if (ok) {
          tmem_fence_after();
          issue_scores(0);
        }
        for (int j = 0; j < n_tiles && ok; ++j) {
          const int stage = j % KV_STAGES, b = j & 1;
          const unsigned phase = (j / 2) & 1;
          if (j + 1 < n_tiles) {
            ok = mbar_wait(&k_full[(j + 1) % KV_STAGES], ((j + 1) / KV_STAGES) & 1, error_flag, 14);
            if (!ok) break;
            tmem_fence_after();
            issue_scores(j + 1);
          }
          ok = mbar_wait(&p_full[b], phase, error_flag, 15) &&
               mbar_wait(&v_full[stage], (j / KV_STAGES) & 1, error_flag, 16);
          if (!ok) break;
          tmem_fence_after();
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            const uint64_t b_desc = umma_desc_mn_major(v_stage(stage) + kk * (16 * 128), BN * 128);
            umma_bf16_a_tmem(tmem_base + o_column, tmem_base + s_column(b) + kk * 8, b_desc, idesc_pv,
                             (j | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&pv_done[j & 1]);
          umma_commit(&kv_empty[stage]);
        }
      }
    } else {
      // ---------------- softmax and output: two threads per query row, one per half of the tile's keys
      const int quarter = warp & 3, half = warp >= 6 ? 1 : 0;
      const int local_row = quarter * 32 + lane;
      const int row = row0 + local_row;
      const int pos = first_pos + row / group;
      const unsigned lane_field = (unsigned)(quarter * 32) << 16;
      const unsigned o_addr = tmem_base + lane_field + o_column + half * (D / 2);     // this thread's half of the output row
      // All 256 threads pass this barrier together; it also tells everyone whether anyone gave up a wait,
      // so that the threads leave the loop together and nobody waits at a barrier alone.
      auto all_ok = [](bool mine) {
        unsigned result;
        asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.and.pred q, 1, 256, p;\nselp.u32 %0, 1, 0, q;\n}"
                     : "=r"(result) : "r"((unsigned)mine) : "memory");
        return result != 0;
      };
      float m_used = -INFINITY;      // the maximum the exponents and the output are currently relative to
      float l = 0.f;                 // the sum over this thread's half of the keys
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        const unsigned phase = (j / 2) & 1;
        const int key0 = tile_begin + j * BN + half * HALF;
        const bool full = (tile_begin + j * BN + BN - 1 <= first_pos + t_lo) &&
                          (window <= 0 || tile_begin + j * BN >= first_pos + t_hi - window + 1);
        ok = ok && mbar_wait(&s_full[b], phase, error_flag, 18);
        ok = __all_sync(0xffffffffu, ok);
        const unsigned s_addr = tmem_base + lane_field + s_column(b) + half * HALF;
        float v[HALF];
        float tile_max = -INFINITY;
        if (ok) {
          tmem_fence_after();
          tmem_load_32_nowait(s_addr, *reinterpret_cast<float(*)[32]>(&v[0]));
          tmem_load_32_nowait(s_addr + 32, *reinterpret_cast<float(*)[32]>(&v[32]));
          tmem_load_wait();
          // eight independent partial maxima (and sums below): a single running value would chain 64 operations
          float part_max[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) part_max[e] = -INFINITY;
          if (full) {
#pragma unroll
            for (int i = 0; i < HALF; ++i) part_max[i & 7] = fmaxf(part_max[i & 7], v[i]);
          } else {
#pragma unroll
            for (int i = 0; i < HALF; ++i) {
              const int key = key0 + i;
              const bool visible = key <= pos && (window <= 0 || key > pos - window);
              if (!visible) v[i] = -INFINITY;
              part_max[i & 7] = fmaxf(part_max[i & 7], v[i]);
            }
          }
          tile_max = fmaxf(fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])),
                           fmaxf(fmaxf(part_max[4], part_max[5]), fmaxf(part_max[6], part_max[7])));
        }
        const __nv_bfloat16 bound = __float2bfloat16_ru(tile_max);
        half_max_s[b][half][local_row] = bound;
        if (!all_ok(ok)) {
          ok = false;
          break;
        }
        tile_max = fmaxf(__bfloat162float(bound), __bfloat162float(half_max_s[b][half ^ 1][local_row]));
        const float candidate = fmaxf(m_used, tile_max);
        // rescale when the maximum has grown by more than 8 in the exponent (or was still -inf)
        const bool grow = candidate != -INFINITY && (m_used == -INFINITY || (candidate - m_used) * scale_log2 > 8.f);
        if (__any_sync(0xffffffffu, grow)) {
          const float factor = grow ? (m_used == -INFINITY ? 0.f : exp2f((m_used - candidate) * scale_log2)) : 1.f;
          if (grow) m_used = candidate;
          l *= factor;
          if (j > 0) {
            ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) / 2) & 1, error_flag, 19);     // the output must be complete up to tile j - 1
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
              tmem_fence_after();
#pragma unroll
              for (int c = 0; c < D / 2; c += 32) {
                float o[32];
                tmem_load_32(o_addr + c, o);
                unsigned scaled[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) scaled[i] = __float_as_uint(o[i] * factor);
                tmem_store_32(o_addr + c, scaled);
              }
              tmem_store_wait();
            }
          }
        }
        if (ok) {
          const float base = m_used == -INFINITY ? 0.f : m_used * scale_log2;
          float part_sum[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) part_sum[e] = 0.f;
#pragma unroll
          for (int c = 0; c < HALF; c += 32) {
            unsigned packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = fast_exp2(v[c + i] * scale_log2 - base);
              const float p1 = fast_exp2(v[c + i + 1] * scale_log2 - base);
              part_sum[(i >> 1) & 7] += p0 + p1;
              const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
              packed[i / 2] = *reinterpret_cast<const unsigned*>(&pair);
            }
            tmem_store_16(tmem_base + lane_field + s_column(b) + (half * HALF + c) / 2, packed);
          }
          const float sum = ((part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3])) +
                            ((part_sum[4] + part_sum[5]) + (part_sum[6] + part_sum[7]));
          tmem_store_wait();
          tmem_fence_before();
          mbar_arrive(&p_full[b]);
          l += sum;
        }
      }
      if (ok && n_tiles > 1) ok = mbar_wait(&pv_done[(n_tiles - 2) & 1], ((n_tiles - 2) / 2) & 1, error_flag, 20);
      if (ok) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) / 2) & 1, error_flag, 20);
      ok = __all_sync(0xffffffffu, ok);
      ok = all_ok(ok);                                 // nobody reads the maxima any more
      float* half_sum_s = reinterpret_cast<float*>(&half_max_s[0][0][0]);      // [half][row]
      half_sum_s[half * ROWS + local_row] = l;
      if (all_ok(ok)) {
        tmem_fence_after();
        l = half_sum_s[local_row] + half_sum_s[ROWS + local_row];      // the same sum in either thread of the row
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = out + ((size_t)(q0 + row / group) * n_q + kv_head * group + row % group) * D + half * (D / 2);
#pragma unroll
        for (int c = 0; c < D / 2; c += 32) {
          float o[32];
          tmem_load_32(o_addr + c, o);
          if (row < rows_total) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 packed;
              __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
              for (int e = 0; e < 4; ++e) pairs[e] = __floats2bfloat162_rn(o[i + 2 * e] * inv, o[i + 2 * e + 1] * inv);
              *reinterpret_cast<uint4*>(dst + c + i) = packed;
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLUMNS) : "memory");
  }
}

static bool encode(CUtensorMap* map, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                   const cuuint32_t* box) {
  EncodeTiled fn = encode_tiled();
  if (fn == nullptr) return false;
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
int launch(const void* q, const void* k_pool, const void* v_pool, int n_pages, const int* block_tables, int table_stride,
           const int* query_start, const int* context_lens, int page_size, int n_q, int n_kv, float scale, int window,
           void* out, int n_requests, int max_query_len, int n_tokens, int* error_flag, cudaStream_t stream) {
  const int group = n_q / n_kv;
  CUtensorMap map_q, map_k, map_v;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_q, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)n_q * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(ROWS / group)};
    MS_REQUIRE(encode(&map_q, 3, q, dims, strides, box), "attention_tcgen05: tensor map of the queries failed");
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n_pages * n_kv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    MS_REQUIRE(encode(&map_k, 2, k_pool, dims, strides, box) && encode(&map_v, 2, v_pool, dims, strides, box),
               "attention_tcgen05: tensor map of the cache pools failed");
  }
  auto kernel = attention_tcgen05_kernel<D>;
  const size_t smem = Layout<D>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("attention_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const long long tiles = ((long long)max_query_len * group + ROWS - 1) / ROWS;
  MS_REQUIRE(tiles <= 65535 && n_requests <= 65535, "attention_tcgen05: grid exceeds the launch limits");
  dim3 grid(n_kv, (unsigned)tiles, n_requests);
  cudaError_t e = ms::launch(kernel, grid, dim3(THREADS), smem, stream, map_q, map_k, map_v, block_tables, table_stride,
                             query_start, context_lens, page_size, n_q, n_kv, scale * 1.4426950408889634f, window,
                             (__nv_bfloat16*)out, error_flag);
  if (e != cudaSuccess) MS_FAIL("attention_tcgen05: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace t5a
}  // namespace ms

using namespace ms;

// Whether this kernel takes the sizes: head size 64 or 128, a group size that divides 128, pages of 8, 16,
// 32, 64 or 128 tokens.
MS_EXPORT int ms_attention_tcgen05_supports(int head_dim, int n_q, int n_kv, int page_size) {
  if (n_kv <= 0 || n_q % n_kv != 0) return 0;
  const int group = n_q / n_kv;
  return (head_dim == 64 || head_dim == 128) && group <= 128 && 128 % group == 0 && page_size >= 8 &&
         page_size <= 128 && 128 % page_size == 0;
}

// Arguments as for ms_paged_attention_mma (one split); n_pages is the number of pages of the pools.
MS_EXPORT int ms_paged_attention_tcgen05(const void* q, const void* k_pool, const void* v_pool, int n_pages,
                                         const int* block_tables, int table_stride, const int* query_start,
                                         const int* context_lens, int page_size, int n_q, int n_kv, int d, float scale,
                                         int window, void* out, int n_requests, int max_query_len, int n_tokens,
                                         int* error_flag, cudaStream_t stream) {
  if (n_tokens == 0 || n_requests == 0) return 0;
  MS_REQUIRE(ms_attention_tcgen05_supports(d, n_q, n_kv, page_size),
             "attention_tcgen05: head size %d, %d/%d heads, page size %d are not taken by this kernel", d, n_q, n_kv, page_size);
  MS_REQUIRE(error_flag != nullptr, "attention_tcgen05: an error flag on the device is required");
  if (d == 128)
    return t5a::launch<128>(q, k_pool, v_pool, n_pages, block_tables, table_stride, query_start, context_lens, page_size,
                            n_q, n_kv, scale, window, out, n_requests, max_query_len, n_tokens, error_flag, stream);
  return t5a::launch<64>(q, k_pool, v_pool, n_pages, block_tables, table_stride, query_start, context_lens, page_size, n_q,
                         n_kv, scale, window, out, n_requests, max_query_len, n_tokens, error_flag, stream);
}
