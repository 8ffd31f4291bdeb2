// out[M, N] = X[M, K] * W[N, K]^T for up to eight rows M (decode steps), without any sum across thread blocks:
// a block owns groups of up to 128 rows of W for the whole of K.
//
//   - the grid is one block per multiprocessor where the weight allows it (16 to 128 rows a block); a block
//     has sixteen computing warps and one that copies: one thread of it issues TMA loads (cp.async.bulk.tensor,
//     128-byte swizzle) of the block's rows into a ring of shared-memory slots, each slot several pieces of
//     64 k (one copy per slot through a three-dimensional map where K is a multiple of 64, else one per
//     piece).  As many slots as the ring holds are requested BEFORE the kernel waits for its predecessor on
//     the stream (no kernel writes weights): for a weight of a few MB that is the block's whole share, which
//     then arrives while the predecessor ends.  The activations (all of X, a few KB, one copy) are requested
//     by the computing side the moment its own wait for the predecessor returns: copies are served in the
//     order of their requests, and asked for by the copying thread after its ring-full of weights they
//     arrived last, 2 us late, though nothing can be multiplied without them;
//   - the computing warps split a piece by k: each reads 16 x 16 parts of W for all of the block's rows and
//     one 16 x 8 part of X with ldmatrix and multiplies them with mma.sync.m16n8k16 (rows of W on the M
//     side, tokens on the N side), float32 accumulation, one independent chain per 16 rows; four warps take
//     the even pieces of a slot and four the odd ones.  Two such teams of eight warps take the ring's slots in
//     turn, each waiting for and freeing its own: what a warp does for a slot is a short chain of waits (the
//     barrier, the loads, the products, the arrival: 0.32 to 0.38 us whatever the slot holds), and with one
//     team that chain was all a multiprocessor could take in, 43 to 50 GB/s, however early the slots had
//     arrived; two chains side by side made a decode step of the 1.7B sizes 3 % faster.  A slot that is used
//     again always comes back to the same team (a wait by the parity of a barrier's phase tells only
//     neighbouring phases apart): the teams take the slots by their count where the ring has an even number
//     of them, by their place in the ring where it is odd.  The sixteen partial sums meet in shared memory at
//     the end.  The number of 16-row tiles per block is a template parameter of that loop: as a variable it
//     leaves every tile's loads and products in the code as branches, and a block with one tile, which has
//     the most pieces to walk, pays for eight;
//   - plain mode stores the 16 x 8 results.  Gated mode expects the weight of a gated feed-forward with its
//     rows in blocks of sixteen, eight of the gate projection followed by the same eight of the up
//     projection, and stores silu(gate) * up for the eight features: the activation costs no kernel and no
//     trip through memory.  (Both factors are rounded to bfloat16 first, as they are where the product and
//     the activation are separate kernels.)
//   - a norm folded into the products around it (decode steps of a pre-norm block: product, residual add, RMSNorm,
//     product).  Residual mode does not store its results: it adds them to the float32 residual stream, stores
//     x' = bfloat16(residual * w) with the weight w of the norm that follows, and leaves the sum of residual^2 over
//     its own columns, per token, in a row of `out_partials` (one row per block).  The product that follows reads
//     x' as its activations and is given those rows: it adds them up in block order, and multiplies its own sums by
//     1 / sqrt(total / size + eps) per token before it stores them (or applies the activation), which is what the
//     norm would have done to its input: (x w) / rms(x) W^T = (x w W^T) / rms(x).  Two kernels fewer per layer,
//     and no block normalises anything twice;
//   - larger products: a weight with more rows than one wave of such blocks takes runs as several waves of
//     blocks of eight tiles, or (on request, see persistent_rows) with one block per multiprocessor that walks
//     group after group of rows through the one ring, its sums meeting in room of their own while the copies
//     for the next group are on their way; activations of more than 96 KB pass through two buffers in parts
//     of K, fetched again for every group of rows (from the L2 cache).  The kernel's second form (MANY) has
//     those loops; the first, for the products of a small model's layers, has them removed at compile time.
//
// Every wait on an mbarrier is bounded: a wait that does not finish within the limit sets the error flag
// that the host checks, and the block drains and returns.
#include "wide_common.cuh"

#include <cstdlib>

namespace ms {
namespace wide {

constexpr int MAX_STAGES = 16;

// The bounded wait in two parts: the first try where it is used, the spinning and the error flag in one place out
// of line.  These kernels run for a few microseconds, and instructions that are seldom needed still have to be
// fetched past.
__device__ __noinline__ bool wait_longer(uint64_t* bar, unsigned parity, int* error_flag, int code) {
  return mbar_wait(bar, parity, error_flag, code);
}
__device__ __forceinline__ bool wait_for(uint64_t* bar, unsigned parity, int* error_flag, int code) {
  return mbar_try_wait(bar, parity) ? true : wait_longer(bar, parity, error_flag, code);
}
constexpr int SMEM_LIMIT = 226 * 1024;       // dynamic shared memory a block may ask for
constexpr int SLOT_TARGET = 16 * 1024;       // a slot is about this large (and two pieces at least)
constexpr int X_WHOLE_LIMIT = 96 * 1024;     // activations up to this size stay in shared memory whole
constexpr int X_PART_TARGET = 48 * 1024;     // larger ones pass through two buffers of about this size

enum : int { MODE_PLAIN = 0, MODE_GATED = 1, MODE_RESIDUAL = 2 };

// A norm folded into the products around it (see the head of this file).
struct Fold {
  const float* in_partials;      // [in_count][X_ROWS], or null: the rows of X are as they should be
  int in_count;
  float inv_size, eps;           // 1 / (columns of X), the norm's eps
  float* residual;               // residual mode: [M, N] float32, updated in place
  const void* norm_weight;       // [N], of the norm that follows
  int norm_dtype;
  __nv_bfloat16* x_next;         // [M, N]
  float* out_partials;           // [blocks][X_ROWS]
};

struct Plan {
  int tiles, pieces, slot_bytes, stages, bulk, smem;
  int groups, grid;                // groups of `tiles` 16-row tiles; blocks (each takes every grid-th group)
  int x_pieces, x_parts, x_bufs;   // 64-k pieces of X held at once, how many such parts K has, buffers for them
  int scratch_bytes;               // room of its own for the partial sums (0: they meet in the ring)
  int odd_ring;                    // slots are used again and their number is odd: see the teams in compute()
  int slots_per_group, part_slots; // ring slots that a group of rows takes in all, and in one full part of K
};

// What one block does, the same arithmetic for the copying thread and the computing warps (the divisions are
// the host's: a kernel of a few microseconds has no time for them).
struct Walk {
  int kc, my_groups, slots_per_group;
  __device__ __forceinline__ Walk(const Plan& plan, int K, bool many) {
    kc = (K + BK - 1) / BK;
    my_groups = many ? (plan.groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 1;
    slots_per_group = plan.slots_per_group;
  }
  __device__ __forceinline__ int part_pieces(const Plan& plan, int part) const { return min(plan.x_pieces, kc - part * plan.x_pieces); }
  __device__ __forceinline__ int part_slots(const Plan& plan, int part) const {
    return part + 1 < plan.x_parts ? plan.part_slots : plan.slots_per_group - (plan.x_parts - 1) * plan.part_slots;
  }
};

// What the computing warps carry along.
struct Consumer {
  uint64_t *full_bar, *empty_bar, *x_full, *x_empty;
  int stages, slot_bytes;
  unsigned ring_u32, x_u32, a_offset, b_offset;
  int warp, lane, half, team;      // half: the even or the odd pieces of a slot; team: the even or the odd slots of the ring
  int* error_flag;
  float* row_scale;                // [X_ROWS] in shared memory: what a token's sums are multiplied by (folded norm)
  float* tile_squares;             // [MAX_TILES][X_ROWS] in shared memory: residual mode's sums of squares per tile
};

// The computing warps' side for blocks of TILES tiles of 16 rows.  For each of the block's groups of rows: the
// parts of K in turn (X for a part waits in its buffer), the part's slots from the ring, then all warps'
// partial sums meet in `scratch` and the warp that owns a tile (warp < TILES) stores it.  A warp waits for and
// frees the slots of its team (every other slot of a group of rows, counted from the group's start, so that the
// k a team sums do not depend on what else the block walks), whether it has a piece in them or not, and only
// counts past the others.  The number of tiles is a template parameter: with it as a variable every tile's loads and
// products stay in the code as branches, and a block of one tile, which has the most pieces to walk, pays for
// eight.
template <int TILES, int MODE, typename OutT, bool MANY>
__device__ __forceinline__ void compute(const Consumer& c, const Plan& plan, const Walk& walk, unsigned char* scratch,
                                        OutT* __restrict__ out, int M, int N, const Fold& fold) {
  constexpr int piece_bytes = TILES * 16 * 128;
  // A folded norm on the input side: the last computing warp adds up the producing blocks' sums of squares, four
  // lanes per token, each taking every fourth block in order, then the four meet in a fixed order.  Nobody needs
  // the result before the sums are stored, so it costs the step nothing.
  if (fold.in_partials != nullptr && c.warp == COMPUTE_WARPS - 1) {
    const int token = c.lane & 7, part = c.lane >> 3;
    float squares = 0.f;
    for (int b = part; b < fold.in_count; b += 4) squares += __ldcg(fold.in_partials + (size_t)b * X_ROWS + token);
    squares += __shfl_xor_sync(0xffffffffu, squares, 8);
    squares += __shfl_xor_sync(0xffffffffu, squares, 16);
    if (c.lane < X_ROWS) c.row_scale[c.lane] = 1.0f / sqrtf(squares * fold.inv_size + fold.eps);
  }
  // Residual mode: what the stored sums are added to is fetched now, while the weights stream
  float held_x = 0.f, held_y = 0.f, held_z = 0.f, held_w = 0.f, norm_lo = 0.f, norm_hi = 0.f;   // as sum.x .. sum.w below
  if (MODE == MODE_RESIDUAL && c.warp < TILES) {
    const int col = ((int)blockIdx.x * TILES + c.warp) * 16 + (c.lane >> 2), t0 = 2 * (c.lane & 3);
    if (col < N) {
      norm_lo = load_as_float(fold.norm_weight, fold.norm_dtype, col);
      if (t0 < M) held_x = __ldcg(fold.residual + (size_t)t0 * N + col);
      if (t0 + 1 < M) held_y = __ldcg(fold.residual + (size_t)(t0 + 1) * N + col);
    }
    if (col + 8 < N) {
      norm_hi = load_as_float(fold.norm_weight, fold.norm_dtype, col + 8);
      if (t0 < M) held_z = __ldcg(fold.residual + (size_t)t0 * N + col + 8);
      if (t0 + 1 < M) held_w = __ldcg(fold.residual + (size_t)(t0 + 1) * N + col + 8);
    }
  }
  int stage = 0, x_seen = 0;                               // the ring's next slot; parts of X waited for so far
  unsigned parity = 0u;                                    // of the phase of that slot's barriers
  bool ok = true;
  float4* partial = reinterpret_cast<float4*>(scratch);    // [warp][tile][lane]
  const int my_groups = MANY ? walk.my_groups : 1, x_parts = MANY ? plan.x_parts : 1;   // (compile-time ones shorten the code)
  for (int gi = 0; gi < my_groups; ++gi) {
    const int group = (int)blockIdx.x + gi * (int)gridDim.x;
    int walked = 0;                                 // slots of this group so far: which team sums which k must not depend on the block's other groups
    float acc[TILES][4];
#pragma unroll
    for (int t = 0; t < TILES; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    for (int part = 0; part < x_parts && ok; ++part) {
      const bool fresh_x = x_parts > 1 || gi == 0;    // X whole in shared memory is fetched once
      const int buf = x_parts > 1 ? x_seen % plan.x_bufs : 0;
      if (fresh_x) {
        ok = wait_for(&c.x_full[buf], (unsigned)(x_seen / plan.x_bufs) & 1u, c.error_flag, 2);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const unsigned x_part = c.x_u32 + (unsigned)(buf * plan.x_pieces * (X_ROWS * 128)) + c.b_offset;
      const int part_pieces = walk.part_pieces(plan, part), slots = walk.part_slots(plan, part);
      for (int slot = 0; slot < slots; ++slot, ++walked) {
        if (((plan.odd_ring ? stage : walked) & 1) == c.team) {   // the other team has the slots in between
          ok = wait_for(&c.full_bar[stage], parity, c.error_flag, 3);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const int piece0 = slot * plan.pieces, pieces = min(plan.pieces, part_pieces - piece0);
          const unsigned w_slot = c.ring_u32 + (unsigned)(stage * c.slot_bytes) + c.a_offset;
          const unsigned x_slot = x_part + (unsigned)(piece0 * (X_ROWS * 128));
          for (int j = c.half; j < pieces; j += 2) {
            unsigned a[TILES][4], b[2];
            ldmatrix_x2(b, x_slot + j * (X_ROWS * 128));
#pragma unroll
            for (int t = 0; t < TILES; ++t) ldmatrix_x4(a[t], w_slot + j * piece_bytes + t * 2048);   // sixteen rows further: the swizzle repeats
#pragma unroll
            for (int t = 0; t < TILES; ++t) mma_16816(acc[t], a[t], b);
          }
          __syncwarp();
          if (c.lane == 0) mbar_arrive(&c.empty_bar[stage]);
        }
        if (++stage == c.stages) {
          stage = 0;
          parity ^= 1u;
        }
      }
      if (fresh_x) {
        if (x_parts > 1 && ok) {                    // the buffer may take the part after next
          __syncwarp();
          if (c.lane == 0) mbar_arrive(&c.x_empty[buf]);
        }
        ++x_seen;
      }
    }
    if (MANY && gi == my_groups - 1) grid_dependency_launch();
    // the partial sums meet (and nobody reads the scratch's last contents any more)
    ok = all_compute_warps(ok);
    if (ok) {
#pragma unroll
      for (int t = 0; t < TILES; ++t) partial[(c.warp * TILES + t) * 32 + c.lane] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    }
    sync_compute_warps();
    if (!ok) return;
    if (c.warp < TILES) {
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < COMPUTE_WARPS; ++w) {
        const float4 p = partial[(w * TILES + c.warp) * 32 + c.lane];
        sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
      }
      // sum.x, sum.y: row (lane / 4) of the warp's tile, tokens 2 (lane % 4) and + 1;  sum.z, sum.w: the row eight further
      const int r = c.lane >> 2, t0 = 2 * (c.lane & 3);
      if (fold.in_partials != nullptr) {            // the folded norm of the input: a factor per token
        const float s0 = c.row_scale[t0], s1 = c.row_scale[t0 + 1];
        sum.x *= s0; sum.z *= s0; sum.y *= s1; sum.w *= s1;
      }
      if (MODE == MODE_RESIDUAL) {
        const int col = (group * TILES + c.warp) * 16 + r;
        float sq0 = 0.f, sq1 = 0.f;                 // of tokens t0 and t0 + 1 over this lane's two columns
        auto settle = [&](bool live, int token, int cc, float before, float add, float w, float& squares) {
          if (!live) return;
          const float v = before + add;
          fold.residual[(size_t)token * N + cc] = v;
          fold.x_next[(size_t)token * N + cc] = __float2bfloat16_rn(v * w);
          squares += v * v;
        };
        settle(col < N && t0 < M, t0, col, held_x, sum.x, norm_lo, sq0);
        settle(col < N && t0 + 1 < M, t0 + 1, col, held_y, sum.y, norm_lo, sq1);
        settle(col + 8 < N && t0 < M, t0, col + 8, held_z, sum.z, norm_hi, sq0);
        settle(col + 8 < N && t0 + 1 < M, t0 + 1, col + 8, held_w, sum.w, norm_hi, sq1);
        // over the tile's sixteen columns (the eight lanes that share lane % 4), in a fixed order
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
          sq0 += __shfl_xor_sync(0xffffffffu, sq0, o);
          sq1 += __shfl_xor_sync(0xffffffffu, sq1, o);
        }
        if (c.lane < 4) {
          c.tile_squares[c.warp * X_ROWS + 2 * c.lane] = sq0;
          c.tile_squares[c.warp * X_ROWS + 2 * c.lane + 1] = sq1;
        }
      } else if (MODE == MODE_GATED) {
        const int feature = (group * TILES + c.warp) * 8 + r, features = N / 2;
        if (feature < features) {
          if (t0 < M) out[(size_t)t0 * features + feature] = from_float<OutT>(silu_times(round_bf16(sum.x), round_bf16(sum.z)));
          if (t0 + 1 < M)
            out[(size_t)(t0 + 1) * features + feature] = from_float<OutT>(silu_times(round_bf16(sum.y), round_bf16(sum.w)));
        }
      } else {
        const int row = (group * TILES + c.warp) * 16 + r;
        if (row < N) {
          if (t0 < M) out[(size_t)t0 * N + row] = from_float<OutT>(sum.x);
          if (t0 + 1 < M) out[(size_t)(t0 + 1) * N + row] = from_float<OutT>(sum.y);
        }
        if (row + 8 < N) {
          if (t0 < M) out[(size_t)t0 * N + row + 8] = from_float<OutT>(sum.z);
          if (t0 + 1 < M) out[(size_t)(t0 + 1) * N + row + 8] = from_float<OutT>(sum.w);
        }
      }
    }
    if (MODE == MODE_RESIDUAL) {                     // the tiles' sums of squares meet, in tile order: one row per block
      sync_compute_warps();
      if (c.warp == 0 && c.lane < X_ROWS) {
        float squares = 0.f;
#pragma unroll
        for (int t = 0; t < TILES; ++t) squares += c.tile_squares[t * X_ROWS + c.lane];
        fold.out_partials[(size_t)blockIdx.x * X_ROWS + c.lane] = squares;
      }
    }
  }
}

// MANY: a block may walk several groups of rows, and K in parts; without it (one group per block, X whole in
// shared memory: the products of a small model's layers) those loops are gone at compile time.
template <int MODE, typename OutT, bool MANY>
__global__ void __launch_bounds__(THREADS, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 OutT* __restrict__ out, int M, int N, int K, const __grid_constant__ Plan plan,
                 const __grid_constant__ Fold fold, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], x_full[2], x_empty[2];
  __shared__ float row_scale[X_ROWS], tile_squares[MAX_TILES * X_ROWS];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = plan.stages, slot_bytes = plan.slot_bytes;
  const Walk walk(plan, K, MANY);
  const int x_buf_bytes = plan.x_pieces * (X_ROWS * 128);
  unsigned char* x_s = smem;                       // x_bufs buffers of x_pieces pieces of [8 tokens x 64 k]
  unsigned char* own_scratch = x_s + (size_t)plan.x_bufs * x_buf_bytes;
  unsigned char* ring = own_scratch + plan.scratch_bytes;

  if (threadIdx.x == 32 * COMPUTE_WARPS) {           // the copying thread's first copies find the maps fetched
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], COMPUTE_WARPS / 2);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&x_full[i], 1);
      mbar_init(&x_empty[i], COMPUTE_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The kernel behind this one may start now if this one is short.  Behind a block that walks many groups it
  // would sit on the multiprocessors for tens of microseconds with its first loads long done, and then run in
  // two waves (measured: a 23 us product took 44 us behind a 40 us one of this kind); such a block lets it
  // start when its own last group is nearly done.
  if (!MANY) grid_dependency_launch();

  if (warp == COMPUTE_WARPS) {
    if (lane == 0) {
      // ---------------- copies: the slots of the block's groups, part of K after part, in one ring
      const int my_groups = MANY ? walk.my_groups : 1, x_parts = MANY ? plan.x_parts : 1;
      const int piece_bytes = plan.tiles * 16 * 128;
      bool ok = true, waited = false;
      int g = 0, stage = 0;                        // the ring's next slot, and the parity of its barriers' phase
      unsigned parity = 0u;
      int x_sent = 1;                              // parts of X requested so far (the first: by the computing side)
      // X comes from the kernel before this one.  Its first part is requested by the computing side the moment
      // that kernel has ended (copies are served in the order of their requests, and behind a ring-full of
      // weights X would arrive last, though it is needed first); later parts are this thread's, which waits
      // for that kernel before the first of them
      auto send_x = [&](int part) {
        if (!waited) {
          grid_dependency_wait();
          waited = true;
        }
        const int buf = x_sent % plan.x_bufs;
        if (x_sent >= plan.x_bufs && !wait_for(&x_empty[buf], ((unsigned)(x_sent / plan.x_bufs) & 1u) ^ 1u, error_flag, 1)) {
          ok = false;
          return;
        }
        if (plan.bulk) {                             // one copy; pieces past the end arrive as zeros and count
          mbar_expect_tx(&x_full[buf], x_buf_bytes);
          tma_load_3d(x_s + (size_t)buf * x_buf_bytes, &map_x, &x_full[buf], 0, 0, part * plan.x_pieces);
        } else {
          const int pieces = walk.part_pieces(plan, part);
          mbar_expect_tx(&x_full[buf], pieces * (X_ROWS * 128));
          for (int i = 0; i < pieces; ++i)
            tma_load_2d(x_s + (size_t)buf * x_buf_bytes + (size_t)i * (X_ROWS * 128), &map_x, &x_full[buf],
                        (part * plan.x_pieces + i) * BK, 0);
        }
        ++x_sent;
      };
      for (int gi = 0; gi < my_groups && ok; ++gi) {
        const int row0 = ((int)blockIdx.x + gi * (int)gridDim.x) * plan.tiles * 16;
        for (int part = 0; part < x_parts && ok; ++part) {
          const bool fresh_x = x_parts > 1 || gi == 0;
          if (fresh_x && (gi > 0 || part > 0)) send_x(part);
          const int part_pieces = walk.part_pieces(plan, part), slots = walk.part_slots(plan, part);
          for (int slot = 0; slot < slots && ok; ++slot, ++g) {
            if (g >= stages && !(ok = wait_for(&empty_bar[stage], parity ^ 1u, error_flag, 1))) break;
            const int piece0 = slot * plan.pieces, pieces = min(plan.pieces, part_pieces - piece0);
            unsigned char* dst = ring + (size_t)stage * slot_bytes;
            if (plan.bulk) {                       // one copy; pieces past the end arrive as zeros and count
              mbar_expect_tx(&full_bar[stage], plan.pieces * piece_bytes);
              tma_load_3d(dst, &map_w, &full_bar[stage], 0, row0, part * plan.x_pieces + piece0);
            } else {
              mbar_expect_tx(&full_bar[stage], pieces * piece_bytes);
              for (int j = 0; j < pieces; ++j)
                tma_load_2d(dst + (size_t)j * piece_bytes, &map_w, &full_bar[stage], (part * plan.x_pieces + piece0 + j) * BK, row0);
            }
            if (++stage == stages) {
              stage = 0;
              parity ^= 1u;
            }
          }
        }
      }
      if (!waited) grid_dependency_wait();
      if (!ok || *reinterpret_cast<volatile int*>(error_flag) != 0) {
        // something gave up: let the copies still in flight land before the block may exit
        for (int j = g - 1; j >= 0 && j >= g - stages; --j) wait_for(&full_bar[j % stages], (j / stages) & 1, error_flag, 4);
        for (int j = x_sent - 1; j >= 0 && j >= x_sent - plan.x_bufs; --j)
          wait_for(&x_full[j % plan.x_bufs], (unsigned)(j / plan.x_bufs) & 1u, error_flag, 4);
      }
    }
    // The other lanes of this warp do nothing, and must not wait for the predecessor here: a warp that
    // waits does so as a whole, and lane 0 would be held back from the loads above.
    return;
  }

  // ---------------- products
  grid_dependency_wait();
  if (threadIdx.x == 0) {                          // the first part of X (all of it, if it fits): see the copying thread
    if (plan.bulk) {
      mbar_expect_tx(&x_full[0], x_buf_bytes);
      tma_load_3d(x_s, &map_x, &x_full[0], 0, 0, 0);
    } else {
      const int pieces = walk.part_pieces(plan, 0);
      mbar_expect_tx(&x_full[0], pieces * (X_ROWS * 128));
      for (int i = 0; i < pieces; ++i) tma_load_2d(x_s + (size_t)i * (X_ROWS * 128), &map_x, &x_full[0], i * BK, 0);
    }
  }
  Consumer c;
  c.full_bar = full_bar;
  c.empty_bar = empty_bar;
  c.x_full = x_full;
  c.x_empty = x_empty;
  c.stages = stages;
  c.slot_bytes = slot_bytes;
  c.ring_u32 = smem_u32(ring);
  c.x_u32 = smem_u32(x_s);
  c.warp = warp;
  c.lane = lane;
  c.half = (warp >> 2) & 1;
  c.team = warp >> 3;
  const int kk = warp & 3;                         // which 16 of a piece's 64 k
  c.a_offset = swizzled((lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4));
  c.b_offset = swizzled(lane & 7, 2 * kk + ((lane >> 3) & 1));
  c.error_flag = error_flag;
  c.row_scale = row_scale;
  c.tile_squares = tile_squares;
  // a block with one group has read every slot when its sums meet, and they meet in the ring; one with more
  // has copies for the next group on their way by then, and room of its own for the sums
  unsigned char* scratch = plan.scratch_bytes > 0 ? own_scratch : ring;
  switch (plan.tiles) {
    case 1: compute<1, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    case 2: compute<2, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    case 3: compute<3, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    case 4: compute<4, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    case 5: compute<5, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    case 6: compute<6, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    case 7: compute<7, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
    default: compute<8, MODE, OutT, MANY>(c, plan, walk, scratch, out, M, N, fold); break;
  }
}

// How the product is laid out; false if it does not fit.  `budget` bounds the shared memory: what a block
// leaves free lets the next kernel's blocks start early, what it takes lets more of the weight be on its way
// before the predecessor has ended.
//   - rows: groups of `tiles` 16-row tiles, dealt to at most one block per multiprocessor; the tile count is the
//     one with which the busiest block has the fewest tiles to walk (a group more per block counts as a tenth
//     of a tile: its sums have to meet once more), the larger count on a draw.  Unless `persistent` is set,
//     a weight with more rows than that gives every block one group runs as several waves of blocks instead;
//   - K: X stays in shared memory whole up to 96 KB; beyond that K is walked in parts of about 48 KB of X
//     through two buffers, for every group again (from the L2 cache);
//   - the ring: slots of about 16 KB (two pieces at least, so that both halves of the warps work), as many as
//     the budget holds.
static bool plan_for(int N, int K, int budget, bool persistent, Plan* plan) {
  if (K <= 0 || N <= 0 || K % 8 != 0) return false;
  const long long sms = multiprocessors();
  const long long kc = (K + BK - 1) / BK;
  const long long row_tiles = ((long long)N + 15) / 16;
  long long tiles = 1;
  double best = 0.0;
  for (long long t = 1; t <= MAX_TILES; ++t) {
    const long long groups = (row_tiles + t - 1) / t, grid = groups < sms ? groups : sms;
    const long long per_block = (groups + grid - 1) / grid;
    const double cost = (double)(per_block * t) + 0.1 * (double)per_block;
    if (t == 1 || cost <= best) {
      best = cost;
      tiles = t;
    }
  }
  long long groups = (row_tiles + tiles - 1) / tiles, grid = groups < sms ? groups : sms;
  if (groups > grid && !persistent && kc * (X_ROWS * 128) <= X_WHOLE_LIMIT) {
    // more rows than one wave of blocks takes: several waves of blocks of eight tiles, one group each
    tiles = MAX_TILES;
    groups = grid = (row_tiles + tiles - 1) / tiles;
  }
  const long long piece_bytes = tiles * 16 * 128;
  long long pieces = SLOT_TARGET / piece_bytes;
  if (pieces < 2) pieces = 2;
  if (pieces > kc) pieces = kc;
  long long x_pieces = kc, x_parts = 1, x_bufs = 1;
  if (kc * (X_ROWS * 128) > X_WHOLE_LIMIT) {
    x_pieces = X_PART_TARGET / (X_ROWS * 128) / pieces * pieces;     // whole slots
    if (x_pieces < pieces) x_pieces = pieces;
    x_parts = (kc + x_pieces - 1) / x_pieces;
    x_bufs = 2;
  }
  const long long slot = pieces * piece_bytes;
  long long slots_per_group = 0;
  for (long long part = 0; part < x_parts; ++part) {
    const long long part_pieces = kc - part * x_pieces < x_pieces ? kc - part * x_pieces : x_pieces;
    slots_per_group += (part_pieces + pieces - 1) / pieces;
  }
  const long long total_slots = slots_per_group * ((groups + grid - 1) / grid);
  const long long x_bytes = x_bufs * x_pieces * (X_ROWS * 128), partial = (long long)COMPUTE_WARPS * tiles * 512;
  const long long scratch = groups > grid ? partial : 0;             // see the kernel: only a block's last sums may meet in the ring
  long long stages = (budget - 1024 - x_bytes - scratch) / slot;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages > total_slots) stages = total_slots;
  // A slot that is used again must come back to the same team of warps: a team waits for its slots by the parity of
  // their barrier's phase, and that tells only neighbouring phases apart.  With an even number of slots in the
  // ring the even ones are always the first team's; with an odd number the teams take the slots by their place in
  // the ring instead of by their count (three of five and two of five, say: uneven, but a ring-ful of 32B q/k/v
  // weights one slot shorter cost more, 1.6 % of a decode step).
  const bool odd_ring = stages < total_slots && stages % 2 != 0;
  if (stages < 2 && stages < total_slots) return false;
  long long ring = stages * slot;
  if (scratch == 0 && ring < partial) ring = partial;
  if (x_bytes + scratch + ring + 1024 > SMEM_LIMIT) return false;
  plan->tiles = (int)tiles;
  plan->pieces = (int)pieces;
  plan->slot_bytes = (int)slot;
  plan->stages = (int)stages;
  plan->bulk = K % BK == 0;
  plan->smem = (int)(x_bytes + scratch + ring + 1024);
  plan->groups = (int)groups;
  plan->grid = (int)grid;
  plan->x_pieces = (int)x_pieces;
  plan->x_parts = (int)x_parts;
  plan->x_bufs = (int)x_bufs;
  plan->scratch_bytes = (int)scratch;
  plan->odd_ring = odd_ring ? 1 : 0;
  plan->slots_per_group = (int)slots_per_group;
  plan->part_slots = (int)((x_pieces + pieces - 1) / pieces);
  return true;
}

static int smem_budget() {
  static int budget = 0;
  if (budget == 0) {
    const char* text = std::getenv("MINISERVE_B200_WIDE_SMEM_KB");
    budget = (text != nullptr && std::atoi(text) >= 32 ? std::atoi(text) : 200) * 1024;
    if (budget > SMEM_LIMIT) budget = SMEM_LIMIT;
  }
  return budget;
}

// Whether blocks walk several groups of rows where the weight has more rows than one wave of blocks takes
// (MINISERVE_B200_WIDE_MANY=1).  Alone that is the fastest of this library's kernels on several large weights, but
// the product that followed it in a decode step of the 8B and 32B sizes took up to twice its usual time, for a
// reason not yet found; several waves of blocks do not have that effect.
static bool persistent_rows() {
  const char* text = std::getenv("MINISERVE_B200_WIDE_MANY");     // read at every call: a test turns it on and off
  return text != nullptr && std::atoi(text) != 0;
}

template <int MODE, typename OutT>
int launch(const void* X, const void* W, void* out, int M, int N, int K, const Fold& fold, int* error_flag, cudaStream_t stream) {
  Plan plan;
  MS_REQUIRE(plan_for(N, K, smem_budget(), persistent_rows(), &plan), "gemm_wide: an inner size of %d leaves no room for the weight ring", K);
  MS_REQUIRE(MODE != MODE_RESIDUAL || (plan.groups <= plan.grid && plan.x_parts == 1),
             "gemm_wide: the residual mode takes weights that one wave of blocks covers, not %d x %d", N, K);
  CUtensorMap map_w, map_x;
  const bool maps_ok = cached_map(&map_w, W, N, K, plan.tiles * 16, plan.bulk ? plan.pieces : 0) && cached_map(&map_x, X, M, K, X_ROWS, plan.bulk ? plan.x_pieces : 0);
  MS_REQUIRE(maps_ok, "gemm_wide: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, N, K);
  const bool many = plan.groups > plan.grid || plan.x_parts > 1;
  auto kernel = (many && MODE != MODE_RESIDUAL) ? gemm_wide_kernel<MODE, OutT, true> : gemm_wide_kernel<MODE, OutT, false>;
  static bool configured[2] = {false, false};
  if (!configured[many]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (e != cudaSuccess) MS_FAIL("gemm_wide: cannot reserve shared memory: %s", cudaGetErrorString(e));
    configured[many] = true;
  }
  cudaError_t e = ms::launch(kernel, dim3(plan.grid), dim3(THREADS), (size_t)plan.smem, stream, map_w, map_x, (OutT*)out, M, N, K,
                             plan, fold, error_flag);
  if (e != cudaSuccess) MS_FAIL("gemm_wide: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace wide
}  // namespace ms

using namespace ms;

// Whether ms_gemm_wide is a candidate for a product of these sizes: 2 with at most one block per multiprocessor
// and the activations whole in shared memory, which is what it was made for first; 1 with more blocks than
// that, or blocks that walk several groups of rows, or K in parts; 0 not offered (ms_gemm_wide itself takes
// every inner size that is a multiple of 8).
MS_EXPORT int ms_gemm_wide_supports(int N, int K) {
  wide::Plan plan;
  if (!wide::plan_for(N, K, wide::smem_budget(), wide::persistent_rows(), &plan)) return 0;
  if (plan.x_parts > 1) return wide::persistent_rows() ? 1 : 0;      // K in parts is offered with the same switch
  return plan.groups <= wide::multiprocessors() ? 2 : 1;
}

// The number of blocks ms_gemm_wide runs for these sizes (the rows of out_partials in its residual mode); 0: not taken.
MS_EXPORT int ms_gemm_wide_blocks(int N, int K) {
  wide::Plan plan;
  return wide::plan_for(N, K, wide::smem_budget(), wide::persistent_rows(), &plan) ? plan.grid : 0;
}

// X [M, K], W [N, K] bfloat16 (K a multiple of 8, both 16-byte aligned), M <= 8.
//   mode 0: out [M, N], bfloat16 (out_dtype 1) or float32 (0);
//   mode 1: W holds a gated feed-forward's gate and up projections in blocks of sixteen rows (eight gate rows,
//           then the up rows of the same eight features; N a multiple of 16); out [M, N / 2] bfloat16 =
//           silu(gate) * up.
// error_flag: one int on the device, zero before the first call; a kernel that gave up waiting writes a
// non-zero code there (1, 4 copies; 2, 3 products), which the caller checks when it synchronises.
//
// A folded norm (see the head of this file).  in_partials [in_count][8] float32 or null: every token's sums are
// multiplied by 1 / sqrt(sum over the rows of in_partials / K + eps) before they are stored.
//   mode 2: nothing is stored to `out` (null); residual [M, N] float32 += the product, x_next [M, N] bfloat16 =
//           residual * norm_weight [N] (float32: norm_dtype 0, bfloat16: 1), out_partials [ms_gemm_wide_blocks(N, K)][8]
//           float32 = sums of residual^2 over each block's columns; only for weights with ms_gemm_wide_supports == 2.
MS_EXPORT int ms_gemm_wide(const void* X, const void* W, void* out, int out_dtype, int mode, int M, int N, int K,
                           const float* in_partials, int in_count, float eps, float* residual, const void* norm_weight,
                           int norm_dtype, void* x_next, float* out_partials, int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  wide::Fold fold = {};
  fold.in_partials = in_count > 0 ? in_partials : nullptr;
  fold.in_count = in_count;
  fold.inv_size = 1.0f / (float)K;
  fold.eps = eps;
  fold.residual = residual;
  fold.norm_weight = norm_weight;
  fold.norm_dtype = norm_dtype;
  fold.x_next = (__nv_bfloat16*)x_next;
  fold.out_partials = out_partials;
  MS_REQUIRE(M <= wide::X_ROWS, "gemm_wide: %d rows; this kernel takes at most %d", M, wide::X_ROWS);
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_wide: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_wide: operands must be 16-byte aligned");
  MS_REQUIRE(error_flag != nullptr, "gemm_wide: an error flag on the device is required");
  if (mode == wide::MODE_GATED) {
    MS_REQUIRE(N % 16 == 0 && out_dtype == MS_BF16, "gemm_wide: gated mode wants a multiple of 16 rows (%d) and bfloat16 results", N);
    return wide::launch<wide::MODE_GATED, __nv_bfloat16>(X, W, out, M, N, K, fold, error_flag, stream);
  }
  if (mode == wide::MODE_RESIDUAL) {
    MS_REQUIRE(residual && norm_weight && x_next && out_partials && (norm_dtype == MS_F32 || norm_dtype == MS_BF16),
               "gemm_wide: the residual mode needs the residual stream, the following norm's weight, x_next and out_partials");
    return wide::launch<wide::MODE_RESIDUAL, __nv_bfloat16>(X, W, nullptr, M, N, K, fold, error_flag, stream);
  }
  MS_REQUIRE(mode == wide::MODE_PLAIN, "gemm_wide: unknown mode %d", mode);
  if (out_dtype == MS_BF16) return wide::launch<wide::MODE_PLAIN, __nv_bfloat16>(X, W, out, M, N, K, fold, error_flag, stream);
  if (out_dtype == MS_F32) return wide::launch<wide::MODE_PLAIN, float>(X, W, out, M, N, K, fold, error_flag, stream);
  MS_FAIL("gemm_wide: unknown output type code %d", out_dtype);
}
