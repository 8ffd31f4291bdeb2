// out[M, N] = X[M, K] * W[N, K]^T for the many-row products of prompt portions, with TWO thread blocks (a cluster
// of two, on neighbouring multiprocessors) working on each 256 x 256 tile of the output: tcgen05.mma with
// cta_group::2.  bfloat16 operands, float32 accumulation in tensor memory.
//
// Each block of a pair loads, for every 64-wide k-block, ITS 128 rows of the X tile and ITS 128 rows of the W tile
// (32 KB; a block working alone on a 128 x 256 tile loads 48 KB for the same number of MMA cycles), and the MMA,
// issued by one thread of the pair's even block, reads both halves of both operands from the two blocks' shared
// memory and accumulates rows 0..127 of the tile in the even block's tensor memory and rows 128..255 in the odd
// block's.  Nothing is loaded for both blocks at once: every block fetches its own halves.
//
// A pair walks over the tiles (pair index, then every (number of pairs)-th; neighbours in this order share their W
// tile).  In the wide form a tile is 256 x 512: the same rows of X meet two W tiles of 256 rows, one accumulator each,
// so that a block loads 48 KB per k-block for twice the MMAs (24 KB per 256 x 256 of work instead of 32 KB: what the
// blocks fetch from the L2 cache is what bounds the kernel); both accumulators are complete together, so only the
// second one's read-out overlaps nothing.  In each block:
//   warp 0      one thread issues the TMA loads of this block's halves into a ring of stages; their arrival is
//               counted on the EVEN block's "full" barrier of the stage;
//   warp 1      allocates tensor memory for two accumulators (both blocks, together); in the even block one thread
//               issues the MMAs and frees each stage with a commit that arrives on the "empty" barrier of BOTH blocks;
//               a last commit per tile announces the accumulator to both blocks' read-out warps;
//   warps 2..5  read this block's 128 rows of the accumulator out of tensor memory, apply the epilogue and store,
//               while the next tile is being accumulated in the other accumulator; then they arrive on the even
//               block's "accumulator free" barrier.  Each warp puts 32 rows x 128 bytes of results at a time into
//               one of its two swizzled 4 KB buffers and hands it to a TMA store (or TMA add), which writes whole
//               lines and clips at the matrix' edges; a thread storing its own row straight from registers
//               touches 32 lines per instruction, and those requests share the path on which the operand loads
//               are asked for.  Output widths that TMA does not take (a row pitch that is no multiple of 16
//               bytes) are stored from registers.
// Epilogues: store (bfloat16 or float32), add into a float32 matrix in place, or the gated activation
// silu(gate) * up of a weight whose rows are paired (eight gate rows, then the same eight up rows).
//
// A norm folded into the products around it, as in the few-row kernel (gemm_wide.cu): the residual epilogue adds its
// results into the float32 stream, stores `stream * norm weight` as bfloat16 and leaves each row's sum of squares
// over the tile's columns in `out_partials [column tiles, M]`; the product that follows (storing or gated) adds
// those up in tile order and multiplies its own results by `1 / sqrt(total / K + eps)` before it rounds them:
// (x w / rms(x)) W^T = (x w) W^T / rms(x).  In that epilogue a read-out warp works on 32 rows x 32 columns at a time:
// the stream's box arrives by TMA in one of two buffers (asked for two boxes ahead, across tiles, so the first ones
// come while the tile is still being accumulated), the results go from tensor memory (a row per thread) through a
// third buffer, and then every instruction handles four whole rows of the box (eight lanes x 16 bytes each), so
// that the stream and the next input are written in whole lines.
//
// The q/k/v epilogue (heads of 128): a thread holds one head of its row at a time (128 accumulators), rounds it to
// bfloat16 as the storing epilogue would and applies the per-head RMSNorm of q and k; the head then goes through
// shared memory to eight lanes per row, which apply the half-split rotation (cosine and sine of the row's position
// from the step's table, read in whole lines) and store q heads to the query matrix and k and v heads to their
// slots of the paged cache, a row's 128 bytes at a time.  That is what the separate norm + rotation + append kernel
// does, without writing the projection out and reading it back.
//
// Every wait on an mbarrier is bounded: a wait that does not finish within the limit sets the error flag that the
// host checks, and the kernel drains and returns (tensor memory is freed on every path; both blocks meet before).
#include "wide_common.cuh"

namespace ms {
namespace pair {

using namespace ms::t5;

constexpr int HALF = 128;                    // rows of X, and rows of W, that one block of the pair loads
constexpr int TILE = 2 * HALF;               // the pair's tile: 256 x 256
constexpr int BK = 64, UMMA_K = 16;
// warps 0 and 1 load and multiply; four read-out warps, or eight in the q/k/v epilogue (a head of the tile for each
// four, two warps per scheduler: the epilogue is long chains of dependent instructions)
__host__ __device__ constexpr int read_warps(int epilogue) { return epilogue == 4 ? 8 : 4; }
__host__ __device__ constexpr int threads(int epilogue) { return 32 * (2 + read_warps(epilogue)); }
constexpr int ACCUMULATORS = 2;
constexpr int OUT_BUFFER = 32 * 128;               // 32 rows x 128 bytes: what one read-out warp stores at a time
// A read-out warp's buffers: two to store from; in the residual epilogue two boxes of the stream and one of results;
// in the q/k/v epilogue 32 rows of a head in bfloat16.
__host__ __device__ constexpr int warp_bytes(int epilogue) { return (epilogue == 3 ? 3 : 2) * OUT_BUFFER; }

enum : int { EPI_STORE = 0, EPI_ADD_F32 = 1, EPI_GATED = 2, EPI_RESIDUAL = 3, EPI_QKV = 4 };
static_assert(warp_bytes(EPI_RESIDUAL) == 3 * OUT_BUFFER, "the residual epilogue has three buffers per warp");

constexpr int HEAD = 128;      // head size of the q/k/v epilogue

// What the q/k/v epilogue needs: N = (n_q + 2 n_kv) * 128 columns, q heads first, then k, then v.
struct Heads {
  const int* slots;             // [M] page * page_size + offset of each row's token (negative: k and v are not stored)
  const void* q_weight;         // [128] norm weights of q and k heads (null: no norm)
  const void* k_weight;
  int weight_dtype;
  float eps;
  const float* cos_sin;         // [M, 64, 2] cosine and sine of each row's position (null: no rotation)
  __nv_bfloat16* k_pool;        // [pages, n_kv, page_size, 128]
  __nv_bfloat16* v_pool;
  int page_size, n_q, n_kv;
};

// What a norm folded into the products needs beside the operands.
struct Fold {
  const float* in_partials;     // [in_count, M] sums of squares left by the product before (or null)
  int in_count;
  float eps;
  const void* norm_weight;      // [N], residual epilogue
  int norm_dtype;
  float* out_partials;          // [column tiles, M], residual epilogue
  float* residual;              // [M, N], residual epilogue
};


using wide::round_bf16;
using wide::silu_times;

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns when at most `Pending` of this thread's bulk groups still read their shared-memory source.
template <int Pending> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// The 16-byte piece `piece` (0..7) of row `row` (0..31) in a 128-byte-swizzled buffer of 32 rows x 128 bytes.
__device__ __forceinline__ uint4* swizzled_piece(unsigned char* buffer, int row, int piece) {
  return reinterpret_cast<uint4*>(buffer + row * 128 + ((piece ^ (row & 7)) << 4));
}

__device__ __forceinline__ void tma_load_box(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  mbar_expect_tx(bar, OUT_BUFFER);
  tma_load_2d(smem_dst, map, bar, x, y);
}

__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 packed;
  __nv_bfloat162* two = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int j = 0; j < 4; ++j) two[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  return packed;
}

template <int STAGES, int EPILOGUE, typename OutT, bool WIDE>
__global__ void __launch_bounds__(threads(EPILOGUE), 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_residual,
                 int through_tma, OutT* __restrict__ out, int M, int N, int K, Fold fold, Heads heads,
                 int* __restrict__ error_flag) {
  static_assert(!(WIDE && EPILOGUE == EPI_RESIDUAL), "the residual epilogue's boxes run on over tiles of 256 columns");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[ACCUMULATORS], acc_empty[ACCUMULATORS];
  __shared__ uint64_t residual_bar[4][2];      // residual epilogue: a read-out warp's two boxes of the stream
  __shared__ unsigned tmem_base_s;
  __shared__ float head_weight[2][HEAD];       // q/k/v epilogue: the norm weights of q and of k heads

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_rank();                 // 0: issues the MMAs
  const int pair_index = (int)cluster_id_x(), pairs = (int)(gridDim.x / 2);
  constexpr int PARTS = WIDE ? 2 : 1;                   // W tiles of 256 rows (accumulators) per tile
  constexpr int STAGE = (1 + PARTS) * HALF * BK * 2;    // this block's rows of X and of each W tile for one k-block
  const int tiles_m = (M + TILE - 1) / TILE, tiles_n = (N + PARTS * TILE - 1) / (PARTS * TILE);
  const int n_tiles = tiles_m * tiles_n;
  const int num_k = (K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);            // the even block's own announcement; both blocks' bytes are counted on it
      mbar_init(&empty_bar[s], 1);           // one commit of the even block's MMA thread
    }
#pragma unroll
    for (int b = 0; b < ACCUMULATORS; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * read_warps(EPILOGUE));      // the read-out warps of both blocks
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) mbar_init(&residual_bar[w >> 1][w & 1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (EPILOGUE == EPI_QKV && warp >= 2 && warp < 6) {
    const int i = threadIdx.x - 64;          // 0..127
    head_weight[0][i] = heads.q_weight ? load_as_float(heads.q_weight, heads.weight_dtype, (size_t)i) : 1.f;
    head_weight[1][i] = heads.k_weight ? load_as_float(heads.k_weight, heads.weight_dtype, (size_t)i) : 1.f;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ACCUMULATORS * TILE) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tmem_fence_before();
  __syncthreads();
  cluster_sync_all();                        // the other block's barriers exist before anything arrives on them
  tmem_fence_after();
  const unsigned tmem_base = tmem_base_s;

  grid_dependency_wait();          // X (and, for the adding epilogue, out) come from earlier kernels
  grid_dependency_launch();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer: this block's halves, one running count of k-blocks over all tiles of the pair
      int it = 0;
      bool ok = true;
      for (int tile = pair_index; tile < n_tiles && ok; tile += pairs) {
        const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
        const int x_row = tile_m * TILE + (int)rank * HALF, w_row = tile_n * PARTS * TILE + (int)rank * HALF;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int stage = it % STAGES;
          const unsigned phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&empty_bar[stage], phase ^ 1, error_flag, 1))) break;
          unsigned char* a_s = smem + (size_t)stage * STAGE;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE);
          const unsigned full = address_in_rank(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(a_s, &map_x, full, kb * BK, x_row);
#pragma unroll
          for (int part = 0; part < PARTS; ++part)
            tma_load_2d_pair(a_s + (1 + part) * HALF * BK * 2, &map_w, full, kb * BK, w_row + part * TILE);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------- MMA issue for the pair
      constexpr unsigned idesc = umma_idesc(TILE, TILE);
      int it = 0, done = 0;
      bool ok = true;
      for (int tile = pair_index; tile < n_tiles && ok; tile += pairs, done += PARTS) {
        // (wide: both accumulators, which the read-out of the tile before frees one after the other)
#pragma unroll
        for (int part = 0; part < PARTS; ++part) {
          const int buf = (done + part) % ACCUMULATORS;
          ok = ok && mbar_wait(&acc_empty[buf], (((done + part) / ACCUMULATORS) & 1) ^ 1, error_flag, 4);
        }
        if (!ok) break;
        tmem_fence_after();
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int stage = it % STAGES;
          const unsigned phase = (it / STAGES) & 1;
          if (!(ok = mbar_wait(&full_bar[stage], phase, error_flag, 2))) break;
          tmem_fence_after();
          unsigned char* a_s = smem + (size_t)stage * STAGE;
          const uint64_t a_desc = umma_desc(a_s);
#pragma unroll
          for (int part = 0; part < PARTS; ++part) {
            const unsigned accumulator = tmem_base + ((done + part) % ACCUMULATORS) * TILE;
            const uint64_t b_desc = umma_desc(a_s + (1 + part) * HALF * BK * 2);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)     // 16 elements (32 bytes) further inside the swizzled row: +2 units
              umma_bf16_pair(accumulator, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);      // both blocks' stage is free once these MMAs have read it
        }
        if (ok) {
#pragma unroll
          for (int part = 0; part < PARTS; ++part)
            umma_commit_pair(&acc_full[(done + part) % ACCUMULATORS]);   // the accumulators are complete in both blocks
        }
      }
    }
  } else {
    // ---------------- read-out: warps 2..5 own the tensor-memory lane quarters 2, 3, 0, 1 of this block
    const int quarter = warp & 3;
    unsigned char* out_s = smem + (size_t)STAGES * STAGE;
    int done = 0, stores = 0;
    bool ok = true;
    unsigned boxes = 0;                      // residual epilogue: boxes of the stream taken so far (they alternate between two buffers)
    if (EPILOGUE == EPI_RESIDUAL && pair_index < n_tiles && lane == 0) {
      // the stream's first two boxes are on the way while the first tile is being accumulated
      for (int b = 0; b < 2; ++b)
        tma_load_box(out_s + quarter * warp_bytes(EPILOGUE) + b * OUT_BUFFER, &map_residual, &residual_bar[quarter][b],
                     (pair_index / tiles_m) * TILE + 32 * b, (pair_index % tiles_m) * TILE + (int)rank * HALF + quarter * 32);
    }
    for (int tile = pair_index; tile < n_tiles && ok; tile += pairs)
    for (int part = 0; part < PARTS; ++part, ++done) {
      // (wide: a tile's two accumulators one after the other, each read out like a tile of 256 columns)
      const int tile_m = tile % tiles_m, tile_n = (tile / tiles_m) * PARTS + part;     // tile_n: in tiles of 256 columns
      const int buf = done % ACCUMULATORS;
      const int row = tile_m * TILE + (int)rank * HALF + quarter * 32 + lane;
      ok = ok && mbar_wait(&acc_full[buf], (done / ACCUMULATORS) & 1, error_flag, 3);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tmem_fence_after();
      const unsigned lanes = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * TILE);
      const int out_row = tile_m * TILE + (int)rank * HALF + quarter * 32;
      // a norm folded in before this product: what is left of it is one factor per row
      float scale = 1.f;
      if (EPILOGUE != EPI_RESIDUAL && EPILOGUE != EPI_ADD_F32 && fold.in_partials != nullptr && row < M) {
        float total = 0.f;
        for (int i = 0; i < fold.in_count; ++i) total += fold.in_partials[(size_t)i * M + row];
        scale = rsqrtf(total / (float)K + fold.eps);
      }
      if (EPILOGUE == EPI_QKV) {
        // A head of the tile for each four warps.  A row per thread first: the head's 128 results are rounded to
        // bfloat16 (as the storing epilogue would), their squares summed (the thread's own sum), and they go as rows of
        // 256 bytes into shared memory (16-byte pieces swizzled by the row's low bits).  Then eight lanes per row:
        // lane j of a row has elements 8 j .. 8 j + 7 and their partners 64 + 8 j .., applies the norm (the row's
        // factor comes by shuffle), reads its 64 bytes of the row's cosines and sines, rotates, and stores two
        // pieces of 16 bytes; four rows per instruction, every row's 128 bytes in one piece.
        const int h = (warp - 2) >> 2;
        const int head = tile_n * (TILE / HEAD) + h;
        if (head < heads.n_q + 2 * heads.n_kv) {
          unsigned char* staging = out_s + (warp - 2) * warp_bytes(EPILOGUE);     // 32 rows x 256 bytes
          const bool is_query = head < heads.n_q, is_value = head >= heads.n_q + heads.n_kv;
          const bool normed = !is_value && (is_query ? heads.q_weight : heads.k_weight) != nullptr;
          float sum_sq = 0.f;
#pragma unroll
          for (int part = 0; part < HEAD / 32; ++part) {
            float v[32];
            tmem_load_32(lanes + (unsigned)(h * HEAD + 32 * part), v);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v[i] = round_bf16(v[i] * scale);
              sum_sq += v[i] * v[i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(staging + lane * 256 + (((4 * part + i) ^ (lane & 7)) << 4)) = pack8(v + 8 * i);
          }
          const float factor = normed ? 1.0f / sqrtf(sum_sq / (float)HEAD + heads.eps) : 1.0f;
          // where this row's k or v head goes, in elements from the pool's start (negative: nowhere)
          long long cache_at = -1;
          if (!is_query && row < M) {
            const int slot = heads.slots[row];
            const int kv_head = head - heads.n_q - (is_value ? heads.n_kv : 0);
            if (slot >= 0)
              cache_at = (((long long)(slot / heads.page_size) * heads.n_kv + kv_head) * heads.page_size + slot % heads.page_size) * HEAD;
          }
          __syncwarp();
          const int group = lane >> 3, j = lane & 7;
          const bool rotate = heads.cos_sin != nullptr && !is_value;
          __nv_bfloat16* pool = is_value ? heads.v_pool : heads.k_pool;
          float wa[8], wb[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            wa[e] = normed ? head_weight[is_query ? 0 : 1][8 * j + e] : 1.f;
            wb[e] = normed ? head_weight[is_query ? 0 : 1][HEAD / 2 + 8 * j + e] : 1.f;
          }
#pragma unroll 2
          for (int pass = 0; pass < 8; ++pass) {
            const int r = 4 * pass + group;
            const long long at = __shfl_sync(0xffffffffu, cache_at, r);
            const float inv = __shfl_sync(0xffffffffu, factor, r);
            const int out_r = out_row + r;
            const unsigned char* from = staging + r * 256;
            const uint4 first = *reinterpret_cast<const uint4*>(from + ((j ^ (r & 7)) << 4));
            const uint4 second = *reinterpret_cast<const uint4*>(from + (((8 + j) ^ (r & 7)) << 4));
            float a[8], b[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 fa = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&first)[e]);
              const float2 fb = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&second)[e]);
              a[2 * e] = fa.x; a[2 * e + 1] = fa.y;
              b[2 * e] = fb.x; b[2 * e + 1] = fb.y;
            }
            if (normed) {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                a[e] = a[e] * inv * wa[e];
                b[e] = b[e] * inv * wb[e];
              }
            }
            if (rotate && out_r < M) {
              const float4* table = reinterpret_cast<const float4*>(heads.cos_sin + (size_t)out_r * HEAD + 16 * j);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const float4 cs = table[q4];              // (cos, sin) of elements 8 j + 2 q4 and 8 j + 2 q4 + 1
                const float a0 = a[2 * q4], b0 = b[2 * q4], a1 = a[2 * q4 + 1], b1 = b[2 * q4 + 1];
                a[2 * q4] = a0 * cs.x - b0 * cs.y;
                b[2 * q4] = b0 * cs.x + a0 * cs.y;
                a[2 * q4 + 1] = a1 * cs.z - b1 * cs.w;
                b[2 * q4 + 1] = b1 * cs.z + a1 * cs.w;
              }
            }
            __nv_bfloat16* dst = nullptr;
            if (is_query) {
              if (out_r < M) dst = reinterpret_cast<__nv_bfloat16*>(out) + ((size_t)out_r * heads.n_q + head) * HEAD;
            } else if (at >= 0) {
              dst = pool + at;
            }
            if (dst != nullptr) {
              *reinterpret_cast<uint4*>(dst + 8 * j) = pack8(a);
              *reinterpret_cast<uint4*>(dst + HEAD / 2 + 8 * j) = pack8(b);
            }
          }
        }
      } else if (EPILOGUE == EPI_RESIDUAL) {
        unsigned char* mine = out_s + quarter * warp_bytes(EPILOGUE);
        unsigned char* results = mine + 2 * OUT_BUFFER;
        const int group = lane >> 3, piece = lane & 7;       // this lane's row of every four, and its 16 bytes of a row
        float squares[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) squares[i] = 0.f;
#pragma unroll 1
        for (int c = 0; c < TILE; c += 32, ++boxes) {
          const int b = boxes & 1;
          unsigned char* stream = mine + b * OUT_BUFFER;
          float v[32];
          tmem_load_32(lanes + (unsigned)c, v);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(swizzled_piece(results, lane, i)) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          ok = mbar_wait(&residual_bar[quarter][b], (boxes >> 1) & 1, error_flag, 5);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          __syncwarp();                                      // every lane's results are in the buffer
          const int col = tile_n * TILE + c + 4 * piece;
          float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
          if (col < N) {
            if (fold.norm_dtype == MS_F32) {
              w = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(fold.norm_weight) + col);
            } else {
              const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(fold.norm_weight) + col);
              const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
              const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
              w = make_float4(lo.x, lo.y, hi.x, hi.y);
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + group;
            const float4 a = *reinterpret_cast<const float4*>(swizzled_piece(results, r, piece));
            float4 t = *reinterpret_cast<const float4*>(swizzled_piece(stream, r, piece));
            t.x += a.x; t.y += a.y; t.z += a.z; t.w += a.w;
            squares[i] += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;       // (what lies beyond N or M is zero)
            const int out_r = out_row + r;
            if (out_r < M && col < N) {
              *reinterpret_cast<float4*>(fold.residual + (size_t)out_r * N + col) = t;
              uint2 next;
              *reinterpret_cast<__nv_bfloat162*>(&next.x) = __floats2bfloat162_rn(t.x * w.x, t.y * w.y);
              *reinterpret_cast<__nv_bfloat162*>(&next.y) = __floats2bfloat162_rn(t.z * w.z, t.w * w.w);
              *reinterpret_cast<uint2*>(out + (size_t)out_r * N + col) = next;
            }
          }
          __syncwarp();                                      // both buffers have been read
          if (lane == 0) {
            // the box after the next: of this tile, or of the pair's next tile
            int next_tile = tile, next_c = c + 64;
            if (next_c >= TILE) {
              next_c -= TILE;
              next_tile += pairs;
            }
            if (next_tile < n_tiles)
              tma_load_box(stream, &map_residual, &residual_bar[quarter][b], (next_tile / tiles_m) * TILE + next_c,
                           (next_tile % tiles_m) * TILE + (int)rank * HALF + quarter * 32);
          }
        }
        if (!ok) break;
        // a row's sums lie in the eight lanes of its group
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float total = squares[i];
          total += __shfl_xor_sync(0xffffffffu, total, 1);
          total += __shfl_xor_sync(0xffffffffu, total, 2);
          total += __shfl_xor_sync(0xffffffffu, total, 4);
          const int out_r = out_row + 4 * i + group;
          if (piece == 0 && out_r < M) fold.out_partials[(size_t)tile_n * M + out_r] = total;
        }
      } else if (through_tma) {
        // 128 bytes of results per row at a time: 64 bfloat16 (from 64 accumulator columns, or 128 for the gated
        // form) or 32 float32
        constexpr int ACC_COLS = EPILOGUE == EPI_GATED ? 128 : sizeof(OutT) == 2 ? 64 : 32;
#pragma unroll 1
        for (int c = 0; c < TILE; c += ACC_COLS, ++stores) {
          unsigned char* buffer = out_s + quarter * warp_bytes(EPILOGUE) + (stores & 1) * OUT_BUFFER;
          if (lane == 0) bulk_wait_read<1>();          // the store that last read this buffer is through with it
          __syncwarp();
#pragma unroll
          for (int part = 0; part < ACC_COLS / 32; ++part) {
            float v[32];
            tmem_load_32(lanes + (unsigned)(c + 32 * part), v);
            if (EPILOGUE == EPI_GATED) {
              // columns 16 j .. 16 j + 7 are gate rows, the next eight the same up rows: 32 columns give 16 results
              // (both rounded to bfloat16 first, as the separate activation kernel finds them)
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float r[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = silu_times(round_bf16(v[16 * h + j] * scale), round_bf16(v[16 * h + 8 + j] * scale));
                *swizzled_piece(buffer, lane, 2 * part + h) = pack8(r);
              }
            } else if (sizeof(OutT) == 2) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= scale;
#pragma unroll
              for (int i = 0; i < 4; ++i) *swizzled_piece(buffer, lane, 4 * part + i) = pack8(v + 8 * i);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                *swizzled_piece(buffer, lane, i) = make_uint4(__float_as_uint(v[4 * i] * scale), __float_as_uint(v[4 * i + 1] * scale),
                                                              __float_as_uint(v[4 * i + 2] * scale), __float_as_uint(v[4 * i + 3] * scale));
            }
          }
          fence_async_shared();
          __syncwarp();
          if (lane == 0) {
            const int x = (tile_n * TILE + c) / (EPILOGUE == EPI_GATED ? 2 : 1);
            if (x < (EPILOGUE == EPI_GATED ? N / 2 : N) && out_row < M) {
              if (EPILOGUE == EPI_ADD_F32) tma_add_2d(&map_out, buffer, x, out_row);
              else tma_store_2d(&map_out, buffer, x, out_row);
            }
            bulk_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < TILE; c += 32) {
          float v[32];
          tmem_load_32(lanes + (unsigned)c, v);
          const int col = tile_n * TILE + c;
          if (row >= M || col >= N) continue;
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= scale;
          if (EPILOGUE == EPI_GATED) {
            OutT* dst = out + (size_t)row * (N / 2) + col / 2;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + 16 * (i >> 3) < N) dst[i] = from_float<OutT>(silu_times(round_bf16(v[16 * (i >> 3) + (i & 7)]), round_bf16(v[16 * (i >> 3) + 8 + (i & 7)])));
          } else if (EPILOGUE == EPI_ADD_F32) {
            float* dst = reinterpret_cast<float*>(out) + (size_t)row * N + col;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < N) dst[i] += v[i];
          } else {
            OutT* dst = out + (size_t)row * N + col;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < N) dst[i] = from_float<OutT>(v[i]);
          }
        }
      }
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_in_cluster(address_in_rank(smem_u32(&acc_empty[buf]), 0));   // may be overwritten
    }
    if (lane == 0) bulk_wait_all();          // this warp's stores have been written before the block ends
  }

  // Nobody leaves, and no tensor memory is freed, while the other block may still read this block's shared
  // memory, write its tensor memory or arrive on its barriers.
  tmem_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ACCUMULATORS * TILE) : "memory");
  }
}

// The output [rows, cols] seen by TMA as boxes of 32 rows x 128 bytes, 128-byte swizzled.  Kept like the operands'
// maps (wide::cached_map): a step's buffers come back at the same addresses.
struct OutKey {
  const void* base;
  int rows, cols, size;
  bool operator==(const OutKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && size == o.size; }
};
struct OutKeyHash {
  size_t operator()(const OutKey& k) const {
    return std::hash<const void*>()(k.base) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 7919u) ^ (size_t)k.size;
  }
};
static bool out_map(CUtensorMap* map, void* base, int rows, int cols, bool float32) {
  static std::mutex mutex;
  static std::unordered_map<OutKey, CUtensorMap, OutKeyHash> cache;
  std::lock_guard<std::mutex> guard(mutex);
  const int size = float32 ? 4 : 2;
  const OutKey key{base, rows, cols, size};
  auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * size};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / size), 32};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, float32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box,
             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

template <int STAGES, int EPILOGUE, typename OutT, bool WIDE = false>
int launch(const void* X, const void* W, void* out, int M, int N, int K, const Fold& fold, float* residual, int* error_flag,
           cudaStream_t stream, const Heads& heads = Heads{}) {
  CUtensorMap map_x, map_w, map_out, map_residual;
  MS_REQUIRE(wide::cached_map(&map_x, X, M, K, HALF) && wide::cached_map(&map_w, W, N, K, HALF),
             "gemm_pair: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, N, K);
  const int out_cols = EPILOGUE == EPI_GATED ? N / 2 : EPILOGUE == EPI_QKV ? heads.n_q * HEAD : N;
  const int through_tma = ((size_t)out_cols * sizeof(OutT)) % 16 == 0 && (uintptr_t)out % 16 == 0;
  map_out = map_residual = map_x;          // (where they are not used)
  if (through_tma && EPILOGUE != EPI_RESIDUAL && EPILOGUE != EPI_QKV)
    MS_REQUIRE(out_map(&map_out, out, M, out_cols, sizeof(OutT) == 4),
               "gemm_pair: cuTensorMapEncodeTiled failed for the output (M %d N %d)", M, out_cols);
  if (EPILOGUE == EPI_RESIDUAL) {
    MS_REQUIRE(through_tma && (uintptr_t)residual % 16 == 0,
               "gemm_pair: the residual epilogue wants N %d a multiple of 8 and 16-byte aligned matrices", N);
    MS_REQUIRE(out_map(&map_residual, residual, M, N, true), "gemm_pair: cuTensorMapEncodeTiled failed for the residual stream");
  }
  auto kernel = gemm_pair_kernel<STAGES, EPILOGUE, OutT, WIDE>;
  const size_t smem = (size_t)STAGES * (WIDE ? 3 : 2) * HALF * BK * 2 + read_warps(EPILOGUE) * warp_bytes(EPILOGUE) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("gemm_pair: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 2;
  }
  const int tile_columns = WIDE ? 2 * TILE : TILE;
  const long long tiles = (long long)((N + tile_columns - 1) / tile_columns) * ((M + TILE - 1) / TILE);
  MS_REQUIRE(tiles <= 1073741823LL, "gemm_pair: %lld tiles in one launch is too many", tiles);
  const long long pairs = tiles < sms / 2 ? tiles : sms / 2;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  config.blockDim = dim3(threads(EPILOGUE), 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // as ms::launch gives every kernel
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, map_x, map_w, map_out, map_residual, through_tma, (OutT*)out, M, N, K, fold, heads, error_flag);
  if (e != cudaSuccess) MS_FAIL("gemm_pair: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace pair
}  // namespace ms

using namespace ms;

// X [M, K], W [N, K] bfloat16 (K a multiple of 8, both 16-byte aligned):
//   epilogue 0: out [M, N] stored as bfloat16 (out_dtype 1) or float32 (out_dtype 0);
//   epilogue 1: added in place into the float32 matrix out [M, N];
//   epilogue 2: W holds eight gate rows, then the same eight up rows, and so on (N a multiple of 16);
//               out [M, N / 2] bfloat16 = silu(gate) * up;
//   epilogue 3: residual [M, N] float32 += the product, in place; out [M, N] bfloat16 = residual * norm_weight
//               (norm_weight [N] of type norm_dtype); out_partials [ms_gemm_pair_column_tiles(N), M] float32
//               receives the rows' sums of squares over each tile's columns (N a multiple of 8).
// in_partials [in_count, M] (epilogues 0 and 2; null: none): sums of squares of X's rows before they were scaled
// by a norm weight; the results are multiplied by 1 / sqrt(total / K + eps) before they are rounded.
// wide != 0 (not with epilogue 3): tiles of 256 x 512 (two accumulators side by side) instead of 256 x 256.
// error_flag: one int on the device, zero before the first call; a kernel that gave up waiting writes a
// non-zero code there (1 producer, 2 MMA issue, 3 read-out, 4 accumulator, 5 residual box), which the caller
// checks when it synchronises.
MS_EXPORT int ms_gemm_pair(const void* X, const void* W, void* out, int out_dtype, int epilogue, int wide, int M, int N, int K,
                           const float* in_partials, int in_count, float eps, float* residual, const void* norm_weight,
                           int norm_dtype, float* out_partials, int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_pair: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_pair: operands must be 16-byte aligned");
  MS_REQUIRE(error_flag != nullptr, "gemm_pair: an error flag on the device is required");
  MS_REQUIRE(in_partials == nullptr || (in_count > 0 && (epilogue == pair::EPI_STORE || epilogue == pair::EPI_GATED)),
             "gemm_pair: row statistics go with the storing and the gated epilogue (count %d, epilogue %d)", in_count, epilogue);
  constexpr int STAGES = 6, STAGES_RESIDUAL = 5, STAGES_WIDE = 4;      // what fits beside the read-out warps' buffers
  const pair::Fold fold{in_partials, in_count, eps, norm_weight, norm_dtype, out_partials, residual};
  if (epilogue == pair::EPI_RESIDUAL) {
    MS_REQUIRE(out_dtype == MS_BF16 && residual != nullptr && norm_weight != nullptr && out_partials != nullptr &&
               (norm_dtype == MS_F32 || norm_dtype == MS_BF16),
               "gemm_pair: the residual epilogue wants a float32 stream, a norm weight, a bfloat16 output and room for the sums");
    return pair::launch<STAGES_RESIDUAL, pair::EPI_RESIDUAL, __nv_bfloat16>(X, W, out, M, N, K, fold, residual, error_flag, stream);
  }
  if (epilogue == pair::EPI_ADD_F32) {
    MS_REQUIRE(out_dtype == MS_F32, "gemm_pair: the adding epilogue works on a float32 matrix");
    return wide ? pair::launch<STAGES_WIDE, pair::EPI_ADD_F32, float, true>(X, W, out, M, N, K, fold, nullptr, error_flag, stream)
                : pair::launch<STAGES, pair::EPI_ADD_F32, float>(X, W, out, M, N, K, fold, nullptr, error_flag, stream);
  }
  if (epilogue == pair::EPI_GATED) {
    MS_REQUIRE(out_dtype == MS_BF16 && N % 16 == 0, "gemm_pair: the gated epilogue stores bfloat16 and wants N %d a multiple of 16", N);
    return wide ? pair::launch<STAGES_WIDE, pair::EPI_GATED, __nv_bfloat16, true>(X, W, out, M, N, K, fold, nullptr, error_flag, stream)
                : pair::launch<STAGES, pair::EPI_GATED, __nv_bfloat16>(X, W, out, M, N, K, fold, nullptr, error_flag, stream);
  }
  MS_REQUIRE(epilogue == pair::EPI_STORE, "gemm_pair: unknown epilogue %d", epilogue);
  if (out_dtype == MS_BF16)
    return wide ? pair::launch<STAGES_WIDE, pair::EPI_STORE, __nv_bfloat16, true>(X, W, out, M, N, K, fold, nullptr, error_flag, stream)
                : pair::launch<STAGES, pair::EPI_STORE, __nv_bfloat16>(X, W, out, M, N, K, fold, nullptr, error_flag, stream);
  if (out_dtype == MS_F32)
    return wide ? pair::launch<STAGES_WIDE, pair::EPI_STORE, float, true>(X, W, out, M, N, K, fold, nullptr, error_flag, stream)
                : pair::launch<STAGES, pair::EPI_STORE, float>(X, W, out, M, N, K, fold, nullptr, error_flag, stream);
  MS_FAIL("gemm_pair: unknown output type code %d", out_dtype);
}

// The q/k/v projection of an attention layer with heads of 128, and what follows it up to the cache: X [M, K],
// W [(n_q + 2 n_kv) * 128, K] bfloat16 (q heads first, then k, then v).  Every head is rounded to bfloat16; q and k
// heads get their RMSNorm (weights [128] of type weight_dtype; null: none) and the half-split rotation by
// cos_sin [M, 64, 2] float32 (null: none); q heads go to q_out [M, n_q * 128], k and v heads to the pools
// [pages, n_kv, page_size, 128] at slots[M] (page * page_size + offset; negative: not stored).  in_partials as above.
MS_EXPORT int ms_gemm_pair_qkv(const void* X, const void* W, void* q_out, int M, int K, const float* in_partials, int in_count,
                               float fold_eps, const int* slots, const void* q_weight, const void* k_weight, int weight_dtype,
                               float eps, const float* cos_sin, void* k_pool, void* v_pool, int page_size, int n_q, int n_kv,
                               int* error_flag, cudaStream_t stream) {
  if (M == 0) return 0;
  const int N = (n_q + 2 * n_kv) * pair::HEAD;
  MS_REQUIRE(n_q > 0 && n_kv > 0 && page_size > 0, "gemm_pair_qkv: %d query heads, %d key/value heads, pages of %d", n_q, n_kv, page_size);
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_pair_qkv: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
             ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) && (cos_sin == nullptr || (uintptr_t)cos_sin % 16 == 0),
             "gemm_pair_qkv: operands, outputs and the rotation table must be 16-byte aligned");
  MS_REQUIRE(slots != nullptr && error_flag != nullptr, "gemm_pair_qkv: slots and an error flag on the device are required");
  MS_REQUIRE(weight_dtype == MS_F32 || weight_dtype == MS_BF16, "gemm_pair_qkv: unknown norm weight type code %d", weight_dtype);
  MS_REQUIRE(in_partials == nullptr || in_count > 0, "gemm_pair_qkv: row statistics of %d tiles", in_count);
  const pair::Fold fold{in_partials, in_count, fold_eps, nullptr, 0, nullptr, nullptr};
  const pair::Heads heads{slots, q_weight, k_weight, weight_dtype, eps, cos_sin, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                          page_size, n_q, n_kv};
  return pair::launch<5, pair::EPI_QKV, __nv_bfloat16>(X, W, q_out, M, N, K, fold, nullptr, error_flag, stream, heads);
}

// Rows of `out_partials` that the residual epilogue writes for a weight of N rows.
MS_EXPORT int ms_gemm_pair_column_tiles(int N) { return (N + pair::TILE - 1) / pair::TILE; }
