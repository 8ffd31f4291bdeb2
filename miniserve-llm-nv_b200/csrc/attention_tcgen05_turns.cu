// Paged grouped-query attention for prompt portions on the fifth-generation tensor cores: the form in which two
// groups of softmax threads take the key tiles in turn.
//
// As in attention_tcgen05.cu a thread block handles 128 query rows of one (request, key/value head), the rows
// being the pairs (token, query head of the kv head's group), token-major, and walks over the keys in tiles of 128.
// There all 256 softmax threads work on every tile, two per row, and a tile's period is their whole chain
// load - maximum - exchange - exponentials - store (about 1,900 cycles, of which the tensor cores need 1,024 for the
// tile's two products and the special-function unit 1,024 for its exponentials).  Here the eight softmax warps are
// two groups of 128 threads, ONE thread per query row, and group g takes the tiles j with j % 2 == g: while one
// group is in the exponentials of tile j, the other is loading and looking at tile j + 1, and the warps that share
// a scheduler belong to different groups.  For that the scores need THREE buffers in tensor memory (the scores of
// tile j + 2 are multiplied while tile j's turn into P and tile j + 1's are being read; with two buffers tile
// j + 2's would have to wait for P V of tile j, and the groups for them), which with the output fills it: columns
// 0..383 scores, 384..384+D output.
//   warps 0, 2   issue TMA loads, one box per cache page: warp 0 the query rows once and the K tiles (a ring of three,
//                free again after the tile's scores), warp 2 the V tiles (a ring of three, free after the tile's
//                output); each runs as far ahead as its ring allows (a tile is on its way for about as long as
//                two tiles take to compute, and K of tile j + 2 is needed when tile j - 1 is done);
//   warps 1, 3   one thread each issues tcgen05.mma: warp 1  S = Q K^T,  as far ahead as the score buffers allow, warp 3
//                O += P V  with P read from tensor memory (written by the softmax threads over the scores it came
//                from) and V as an MN-major operand.  (An issuing thread stands still while the tensor cores work on
//                what it has issued; one thread for both kinds took 2,350 cycles a tile for 1,400 cycles of MMAs.)
//   warps 4..7   softmax of the even tiles, warps 8..11 of the odd tiles (a warp reaches its own quarter of the
//                tensor-memory lanes): read the row of S, mask by absolute position, fix the row's maximum, write P
//                as bfloat16.  What the groups share is the row's running maximum: the group of tile j leaves it in
//                shared memory as soon as it has seen its scores, and the group of tile j + 1 waits for it before
//                it fixes its own.  The output in tensor memory is rescaled (by the group that finds it) only when
//                a row's maximum has grown by more than 2^8 since the last rescale.  Each group keeps its own sum,
//                relative to the maximum it last used; at the end the two are brought to the final maximum and
//                added, and each of a row's two threads divides and stores half of the output's columns.
// A softmax thread holds a whole row of 128 scores: those warps take 232 registers each (setmaxnreg) and the first
// four warps give theirs back (40).
// All mbarrier waits are bounded; a wait that runs out sets the error flag and every role drains and returns.
#include "tcgen05.cuh"

namespace ms {
namespace t5c {

using namespace ms::t5;

constexpr int ROWS = 128, BN = 128, THREADS = 384, TMEM_COLUMNS = 512, S_BUFFERS = 3, K_STAGES = 3, V_STAGES = 3;

// 2^x by the special-function unit (ex2.approx): relative error about 2^-22, -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct Layout {
  static constexpr int DBLOCKS = D / 64;                 // 128-byte column blocks of a row
  static constexpr int Q_BYTES = ROWS * D * 2;
  static constexpr int TILE_BYTES = BN * D * 2;          // one K or V tile
  static constexpr size_t TOTAL = (size_t)Q_BYTES + (size_t)(K_STAGES + V_STAGES) * TILE_BYTES + 1024;
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_turns_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_out,
                       const int* __restrict__ block_tables, int table_stride,
                       const int* __restrict__ query_start, const int* __restrict__ context_lens, int page_size, int n_q,
                       int n_kv, float scale_log2, int window, __nv_bfloat16* __restrict__ out, int* __restrict__ error_flag) {
  using L = Layout<D>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  auto k_stage = [&](int s) { return smem + L::Q_BYTES + (size_t)s * L::TILE_BYTES; };
  auto v_stage = [&](int s) { return smem + L::Q_BYTES + (size_t)(K_STAGES + s) * L::TILE_BYTES; };
  __shared__ uint64_t q_full, k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
  __shared__ uint64_t s_full[S_BUFFERS], p_full[S_BUFFERS];
  // pv_done[j & 1]: the output is complete up to key tile j.  A wait by parity only tells the completion that comes
  // next from the one before it: whoever waits for tile j's must know that tile j - 2's has happened AND that tile
  // j + 2's cannot have (a waiter that comes too late sees the parity it waits for flipped back, and waits for good).
  // Only the softmax groups' wait for tile j - 1's output at tile j is of that kind (they have seen tile j's scores,
  // which came behind tile j - 3's output, and tile j + 1 needs their own maxima first).  The score buffers are
  // handed back through s_free[buffer], which like every ring here cannot run ahead of its waiter; the end of all
  // outputs has a barrier of its own, all_done.
  __shared__ uint64_t pv_done[2], s_free[S_BUFFERS], all_done;
  __shared__ uint64_t m_ready[2];              // the rows' maxima after an even / an odd tile are in place
  __shared__ float m_shared[ROWS];
  __shared__ float sums[2][ROWS];              // the two groups' sums, at the end
  __shared__ unsigned tmem_base_s;

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
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
#pragma unroll
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
#pragma unroll
    for (int b = 0; b < S_BUFFERS; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], ROWS);
      mbar_init(&s_free[b], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&pv_done[b], 1);
      mbar_init(&m_ready[b], ROWS);
    }
    mbar_init(&all_done, 1);
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
  const unsigned o_column = S_BUFFERS * BN;

  grid_dependency_wait();
  grid_dependency_launch();

  // The warps that load and multiply, and two idle ones, give registers back, and the softmax warps take them; each
  // side's code lies behind its own setmaxnreg.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (active && (warp == 0 || warp == 2)) {
      // ---------------- producers: lane 0 announces the bytes, all lanes issue the page loads
      const bool keys = warp == 0;
      if (keys && lane == 0) {
        mbar_expect_tx(&q_full, L::Q_BYTES);
#pragma unroll
        for (int db = 0; db < L::DBLOCKS; ++db)
          tma_load_3d(q_s + db * (ROWS * 128), &map_q, &q_full, db * 64, kv_head * group, q0 + t_lo);
      }
      const int pages_per_tile = BN / page_size;
      const int loads_per_tile = pages_per_tile * L::DBLOCKS;
      const int stages = keys ? K_STAGES : V_STAGES;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % stages;
        const unsigned phase = (j / stages) & 1;
        uint64_t* empty = keys ? &k_empty[stage] : &v_empty[stage];
        uint64_t* full = keys ? &k_full[stage] : &v_full[stage];
        if (lane == 0) {
          ok = mbar_wait(empty, phase ^ 1, error_flag, 11);
          if (ok) mbar_expect_tx(full, L::TILE_BYTES);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const int key0 = tile_begin + j * BN;
        unsigned char* to = keys ? k_stage(stage) : v_stage(stage);
        for (int i = lane; i < loads_per_tile; i += 32) {
          const int p = i / L::DBLOCKS, db = i % L::DBLOCKS;
          const int key = key0 + p * page_size;
          // pages past the context are replaced by the request's first page: finite numbers that the mask removes
          const int page = key < key_end ? table[key / page_size] : table[0];
          const int pool_row = (page * n_kv + kv_head) * page_size;
          const size_t at = (size_t)db * (BN * 128) + (size_t)(p * page_size) * 128;
          tma_load_2d(to + at, keys ? &map_k : &map_v, full, db * 64, pool_row);
        }
      }
    } else if (active && warp == 1 && lane == 0) {
      // ---------------- MMA issue, scores.  An issuing thread stands still while the tensor cores work on what it
      // has issued, so the two kinds of product have a thread each: this one runs ahead as far as the three score
      // buffers allow (the buffer of tile j held P of tile j - 3, and is free when that tile's output is complete).
      // The operand descriptors are made once (a stage's differ from the first stage's by its offset in 16-byte
      // units, a k step's by a constant), so that an MMA costs an addition or two: the thread shares its scheduler
      // with two softmax warps.
      constexpr unsigned idesc_s = umma_idesc(ROWS, BN, false);
      constexpr uint64_t TILE_UNITS = L::TILE_BYTES / 16, BLOCK_UNITS = (BN * 128) / 16;
      const uint64_t q_desc = umma_desc(q_s), k_desc = umma_desc(k_stage(0));
      bool ok = mbar_wait(&q_full, 0, error_flag, 12);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % K_STAGES, b = j % S_BUFFERS;
        if (j >= S_BUFFERS) ok = mbar_wait(&s_free[b], (unsigned)(j / S_BUFFERS - 1) & 1u, error_flag, 13);
        ok = ok && mbar_wait(&k_full[stage], (j / K_STAGES) & 1, error_flag, 14);
        if (!ok) break;
        tmem_fence_after();
        const uint64_t keys = k_desc + (uint64_t)stage * TILE_UNITS;
        const unsigned scores = tmem_base + s_column(b);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(scores, q_desc + (kk / 4) * BLOCK_UNITS + 2 * (kk % 4), keys + (kk / 4) * BLOCK_UNITS + 2 * (kk % 4), idesc_s,
                    kk != 0 ? 1u : 0u);
        umma_commit(&s_full[b]);
        umma_commit(&k_empty[stage]);         // the K stage is free again once they are done
      }
    } else if (active && warp == 3 && lane == 0) {
      // ---------------- MMA issue, outputs
      constexpr unsigned idesc_pv = umma_idesc(ROWS, D, true);
      constexpr uint64_t TILE_UNITS = L::TILE_BYTES / 16;
      const uint64_t v_desc = umma_desc_mn_major(v_stage(0), BN * 128);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % V_STAGES, b = j % S_BUFFERS;
        ok = mbar_wait(&p_full[b], (j / S_BUFFERS) & 1, error_flag, 15) &&
             mbar_wait(&v_full[stage], (j / V_STAGES) & 1, error_flag, 16);
        if (!ok) break;
        tmem_fence_after();
        const uint64_t values = v_desc + (uint64_t)stage * TILE_UNITS;
        const unsigned p = tmem_base + s_column(b);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)      // sixteen keys further: 16 rows of 128 bytes in V, 8 columns of packed P
          umma_bf16_a_tmem(tmem_base + o_column, p + kk * 8, values + kk * (16 * 128 / 16), idesc_pv, (j | kk) != 0 ? 1u : 0u);
        umma_commit(&pv_done[j & 1]);
        umma_commit(&s_free[b]);              // (P of this tile is consumed: its buffer may take the scores of tile j + 3)
        umma_commit(&v_empty[stage]);
        if (j == n_tiles - 1) umma_commit(&all_done);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    if (active) {
      // ---------------- softmax and output: one thread per query row, the two groups take the key tiles in turn
      const int quarter = warp & 3, turn = warp >= 8 ? 1 : 0;
      const int local_row = quarter * 32 + lane;
      const int row = row0 + local_row;
      const int pos = first_pos + row / group;
      const unsigned lane_field = (unsigned)(quarter * 32) << 16;
      const unsigned o_addr = tmem_base + lane_field + o_column;
      float m_mine = -INFINITY;      // the maximum this thread's sum is relative to
      float l = 0.f;                 // the sum over this group's tiles
      bool ok = true;
      for (int j = turn; j < n_tiles; j += 2) {
        const int b = j % S_BUFFERS;
        const unsigned s_addr = tmem_base + lane_field + s_column(b);
        const int key0 = tile_begin + j * BN;
        const bool full = (key0 + BN - 1 <= first_pos + t_lo) && (window <= 0 || key0 >= first_pos + t_hi - window + 1);
        ok = ok && mbar_wait(&s_full[b], (j / S_BUFFERS) & 1, error_flag, 18);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tmem_fence_after();
        float v[BN];
#pragma unroll
        for (int c = 0; c < BN; c += 32) tmem_load_32_nowait(s_addr + c, *reinterpret_cast<float(*)[32]>(&v[c]));
        tmem_load_wait();
        // eight independent partial maxima (and sums below): a single running value would chain 128 operations
        float part_max[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) part_max[e] = -INFINITY;
        if (full) {
#pragma unroll
          for (int i = 0; i < BN; ++i) part_max[i & 7] = fmaxf(part_max[i & 7], v[i]);
        } else {
          // key key0 + i is visible to this row if first <= i <= last (causal: last = pos - key0; a window cuts
          // below): one subtraction and one unsigned comparison per score
          const int last = pos - key0;
          const int first = window > 0 ? max(0, pos - window + 1 - key0) : 0;
          const int below = last >= first ? -first : -(1 << 20);           // (nothing visible: no i passes)
          const unsigned span = last >= first ? (unsigned)(last - first) : 0u;
#pragma unroll
          for (int i = 0; i < BN; ++i) {
            if ((unsigned)(i + below) > span) v[i] = -INFINITY;
            part_max[i & 7] = fmaxf(part_max[i & 7], v[i]);
          }
        }
        const float tile_max = fmaxf(fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])),
                                     fmaxf(fmaxf(part_max[4], part_max[5]), fmaxf(part_max[6], part_max[7])));
        // the maximum in use after the tile before (which the other group has worked on, or is still working on)
        float m_used = -INFINITY;
        if (j > 0) {
          ok = mbar_wait(&m_ready[turn ^ 1], ((j - 1) / 2) & 1, error_flag, 21);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          m_used = m_shared[local_row];
        }
        const float candidate = fmaxf(m_used, tile_max);
        // the output is rescaled when the maximum has grown by more than 8 in the exponent (or was still -inf)
        const bool grow = candidate != -INFINITY && (m_used == -INFINITY || (candidate - m_used) * scale_log2 > 8.f);
        if (__any_sync(0xffffffffu, grow)) {
          const float factor = grow ? (m_used == -INFINITY ? 0.f : exp2f((m_used - candidate) * scale_log2)) : 1.f;
          if (j > 0) {
            // the output must be complete up to tile j - 1 (tile j - 3's is: this tile's scores came behind it)
            ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) / 2) & 1, error_flag, 19);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tmem_fence_after();
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
              float o[32];
              tmem_load_32(o_addr + c, o);
              unsigned scaled[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) scaled[i] = __float_as_uint(o[i] * factor);
              tmem_store_32(o_addr + c, scaled);
            }
            tmem_store_wait();
          }
          if (grow) m_used = candidate;
        }
        m_shared[local_row] = m_used;
        mbar_arrive(&m_ready[turn]);               // (the group of tile j + 1 may go on)
        // this group's sum follows the maximum in use
        if (m_used != m_mine) {
          l *= m_mine == -INFINITY ? 0.f : exp2f((m_mine - m_used) * scale_log2);
          m_mine = m_used;
        }
        const float base = m_used == -INFINITY ? 0.f : m_used * scale_log2;
        float part_sum[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) part_sum[e] = 0.f;
#pragma unroll
        for (int c = 0; c < BN; c += 32) {
          unsigned packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = fast_exp2(v[c + i] * scale_log2 - base);
            const float p1 = fast_exp2(v[c + i + 1] * scale_log2 - base);
            part_sum[(i >> 1) & 7] += p0 + p1;
            const __nv_bfloat162 two = __floats2bfloat162_rn(p0, p1);
            packed[i / 2] = *reinterpret_cast<const unsigned*>(&two);
          }
          tmem_store_16(s_addr + c / 2, packed);
        }
        tmem_store_wait();
        tmem_fence_before();
        mbar_arrive(&p_full[b]);
        l += ((part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3])) + ((part_sum[4] + part_sum[5]) + (part_sum[6] + part_sum[7]));
      }
      // All 256 threads pass these barriers together; they also tell everyone whether anyone gave up a wait.
      auto all_ok = [](bool mine) {
        unsigned result;
        asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 p, %1, 0;\nbar.red.and.pred q, 1, 256, p;\nselp.u32 %0, 1, 0, q;\n}"
                     : "=r"(result) : "r"((unsigned)mine) : "memory");
        return result != 0;
      };
      // every output is complete (a barrier that completes once: nothing to tell apart)
      if (ok) ok = mbar_wait(&all_done, 0u, error_flag, 20);
      ok = __all_sync(0xffffffffu, ok);
      ok = all_ok(ok);                  // every maximum is final
      const float m_final = m_shared[local_row];
      if (m_mine != m_final) l *= m_mine == -INFINITY ? 0.f : exp2f((m_mine - m_final) * scale_log2);
      sums[turn][local_row] = l;
      if (all_ok(ok)) {
        tmem_fence_after();
        l = sums[0][local_row] + sums[1][local_row];                  // the same sum in either thread of the row
        const float inv = l > 0.f ? 1.f / l : 0.f;
        // Each of the row's two threads takes half of its columns.  A whole tile goes through the shared memory of
        // the queries (no longer needed; the same layout) and leaves by TMA in whole lines: a thread storing its
        // own row touches 32 lines per instruction, 1,700 cycles for the tile.  A tile that the request's rows do not
        // fill is stored by its threads (what lies behind the rows belongs to the next request).
        const bool whole = row0 + ROWS <= rows_total;
        __nv_bfloat16* dst = out + ((size_t)(q0 + row / group) * n_q + kv_head * group + row % group) * D + turn * (D / 2);
#pragma unroll 1
        for (int c = 0; c < D / 2; c += 32) {
          float o[32];
          tmem_load_32(o_addr + turn * (D / 2) + c, o);
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int e = 0; e < 4; ++e) pairs[e] = __floats2bfloat162_rn(o[i + 2 * e] * inv, o[i + 2 * e + 1] * inv);
            if (whole) {
              const int column = turn * (D / 2) + c + i;          // of the row: 128-byte block column / 64, 16-byte piece within
              *reinterpret_cast<uint4*>(q_s + (column / 64) * (ROWS * 128) + local_row * 128 + ((((column % 64) / 8) ^ (local_row & 7)) << 4)) = packed;
            } else if (row < rows_total) {
              *reinterpret_cast<uint4*>(dst + c + i) = packed;
            }
          }
        }
        if (whole) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          all_ok(true);                                   // the tile is in shared memory
          if (warp == 4 && lane == 0) {
#pragma unroll
            for (int db = 0; db < L::DBLOCKS; ++db)
              asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                           ::"l"(reinterpret_cast<uint64_t>(&map_out)), "r"(smem_u32(q_s + db * (ROWS * 128))), "r"(db * 64),
                             "r"(kv_head * group), "r"(q0 + t_lo) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // shared memory has been read before the block ends
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
  CUtensorMap map_q, map_k, map_v, map_out;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_q, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)n_q * D * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(ROWS / group)};
    MS_REQUIRE(encode(&map_q, 3, q, dims, strides, box) && encode(&map_out, 3, out, dims, strides, box),
               "attention_turns: tensor map of the queries or of the output failed");
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)n_pages * n_kv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    MS_REQUIRE(encode(&map_k, 2, k_pool, dims, strides, box) && encode(&map_v, 2, v_pool, dims, strides, box),
               "attention_turns: tensor map of the cache pools failed");
  }
  auto kernel = attention_turns_kernel<D>;
  const size_t smem = Layout<D>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("attention_turns: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const long long tiles = ((long long)max_query_len * group + ROWS - 1) / ROWS;
  MS_REQUIRE(tiles <= 65535 && n_requests <= 65535, "attention_turns: grid exceeds the launch limits");
  dim3 grid(n_kv, (unsigned)tiles, n_requests);
  cudaError_t e = ms::launch(kernel, grid, dim3(THREADS), smem, stream, map_q, map_k, map_v, map_out, block_tables, table_stride,
                             query_start, context_lens, page_size, n_q, n_kv, scale * 1.4426950408889634f, window,
                             (__nv_bfloat16*)out, error_flag);
  if (e != cudaSuccess) MS_FAIL("attention_turns: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace t5c
}  // namespace ms

using namespace ms;

// Arguments and sizes as for ms_paged_attention_tcgen05 (ms_attention_tcgen05_supports answers for both).
MS_EXPORT int ms_paged_attention_turns(const void* q, const void* k_pool, const void* v_pool, int n_pages,
                                       const int* block_tables, int table_stride, const int* query_start,
                                       const int* context_lens, int page_size, int n_q, int n_kv, int d, float scale,
                                       int window, void* out, int n_requests, int max_query_len, int n_tokens,
                                       int* error_flag, cudaStream_t stream) {
  if (n_tokens == 0 || n_requests == 0) return 0;
  const int group = n_kv > 0 && n_q % n_kv == 0 ? n_q / n_kv : 0;
  MS_REQUIRE((d == 64 || d == 128) && group > 0 && group <= 128 && 128 % group == 0 && page_size >= 8 && page_size <= 128 &&
             128 % page_size == 0,
             "attention_turns: head size %d, %d/%d heads, page size %d are not taken by this kernel", d, n_q, n_kv, page_size);
  MS_REQUIRE(error_flag != nullptr, "attention_turns: an error flag on the device is required");
  if (d == 128)
    return t5c::launch<128>(q, k_pool, v_pool, n_pages, block_tables, table_stride, query_start, context_lens, page_size,
                            n_q, n_kv, scale, window, out, n_requests, max_query_len, n_tokens, error_flag, stream);
  return t5c::launch<64>(q, k_pool, v_pool, n_pages, block_tables, table_stride, query_start, context_lens, page_size, n_q,
                         n_kv, scale, window, out, n_requests, max_query_len, n_tokens, error_flag, stream);
}
