// out[M, N] = X[M, K] * W[N, K]^T for up to eight rows M (decode steps) and a weight with many rows, without
// any sum across thread blocks: a block owns up to 128 rows of W for the whole of K.
//
//   - the grid is one block per multiprocessor where the weight allows it (16 to 128 rows a block); a block
//     has eight computing warps and one that copies: one thread of it issues TMA loads (cp.async.bulk.tensor,
//     128-byte swizzle) of the block's rows into a ring of shared-memory slots, each slot several pieces of
//     64 k (one copy per slot through a three-dimensional map where K is a multiple of 64, else one per
//     piece).  As many slots as the ring holds are requested BEFORE the kernel waits for its predecessor on
//     the stream (no kernel writes weights): for a weight of a few MB that is the block's whole share, which
//     then arrives while the predecessor ends.  The activations (all of X, a few KB) follow after the wait;
//   - the computing warps split a piece by k: each reads 16 x 16 parts of W for all of the block's rows and
//     one 16 x 8 part of X with ldmatrix and multiplies them with mma.sync.m16n8k16 (rows of W on the M
//     side, tokens on the N side), float32 accumulation, one independent chain per 16 rows; four warps take
//     the even pieces of a slot and four the odd ones; every warp waits for every slot and frees it.  The
//     eight partial sums meet in shared memory at the end.  The number of 16-row tiles per block is a
//     template parameter of that loop: as a variable it leaves every tile's loads and products in the code
//     as branches, and a block with one tile, which has the most pieces to walk, pays for eight;
//   - plain mode stores the 16 x 8 results.  Gated mode expects the weight of a gated feed-forward with its
//     rows in blocks of sixteen, eight of the gate projection followed by the same eight of the up
//     projection, and stores silu(gate) * up for the eight features: the activation costs no kernel and no
//     trip through memory.  (Both factors are rounded to bfloat16 first, as they are where the product and
//     the activation are separate kernels.)
//
// Every wait on an mbarrier is bounded: a wait that does not finish within the limit sets the error flag
// that the host checks, and the block drains and returns.
#include "wide_common.cuh"

#include <cstdlib>

namespace ms {
namespace wide {

constexpr int MAX_STAGES = 16;
constexpr int SMEM_LIMIT = 226 * 1024;       // dynamic shared memory a block may ask for
constexpr int SLOT_TARGET = 16 * 1024;       // a slot is about this large (and two pieces at least)

enum : int { MODE_PLAIN = 0, MODE_GATED = 1 };

struct Plan {
  int tiles, pieces, slot_bytes, stages, bulk, smem;
};

struct Phase {
  int tiles, pieces, slots, kc;    // 16-row tiles per block, 64-k pieces per slot, slots, pieces in all
};

// What the computing warps carry through both products.
struct Consumer {
  uint64_t *full_bar, *empty_bar;
  int stages, slot_bytes;
  unsigned ring_u32, a_offset, b_offset;
  int warp, lane, group;
  int* error_flag;
  int stage;                       // of the ring's next slot, and the parity of its barrier's phase
  unsigned parity;
  bool ok;
};

// One product's share of a block: TILES tiles of 16 rows of W over the whole inner size, read from the ring
// slot after slot; the warps' partial sums meet in `scratch`, and the warp that owns a tile (warp < TILES)
// gets its sums back in `sum`.  Every computing warp waits for every slot and frees it, whether it has a
// piece in it or not, so all of them see every phase of a slot's barriers.  The number of tiles is a
// template parameter: with it as a variable every tile's loads and products stay in the code as branches,
// and a product of one tile per block, which has the most pieces to walk, pays for eight.
template <int TILES>
__device__ __forceinline__ void product_tiles(Consumer& c, const Phase& phase, int slots, unsigned x_u32,
                                              unsigned char* scratch, float4& sum) {
  float acc[TILES][4];
#pragma unroll
  for (int t = 0; t < TILES; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
  constexpr int piece_bytes = TILES * 16 * 128;
  for (int slot = 0; slot < slots && c.ok; ++slot) {
    c.ok = mbar_wait(&c.full_bar[c.stage], c.parity, c.error_flag, 3);
    c.ok = __all_sync(0xffffffffu, c.ok);
    if (!c.ok) break;
    const int piece0 = slot * phase.pieces, pieces = min(phase.pieces, phase.kc - piece0);
    const unsigned w_slot = c.ring_u32 + (unsigned)(c.stage * c.slot_bytes) + c.a_offset;
    const unsigned x_slot = x_u32 + (unsigned)(piece0 * (X_ROWS * 128)) + c.b_offset;
    for (int j = c.group; j < pieces; j += 2) {
      unsigned a[TILES][4], b[2];
      ldmatrix_x2(b, x_slot + j * (X_ROWS * 128));
#pragma unroll
      for (int t = 0; t < TILES; ++t) ldmatrix_x4(a[t], w_slot + j * piece_bytes + t * 2048);   // sixteen rows further: the swizzle repeats
#pragma unroll
      for (int t = 0; t < TILES; ++t) mma_16816(acc[t], a[t], b);
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive(&c.empty_bar[c.stage]);
    if (++c.stage == c.stages) {
      c.stage = 0;
      c.parity ^= 1u;
    }
  }
  c.ok = all_compute_warps(c.ok);                          // (also: nobody reads the scratch's old contents any more)
  float4* partial = reinterpret_cast<float4*>(scratch);    // [warp][tile][lane]
  if (c.ok) {
#pragma unroll
    for (int t = 0; t < TILES; ++t) partial[(c.warp * TILES + t) * 32 + c.lane] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
  }
  sync_compute_warps();
  sum = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c.ok && c.warp < TILES) {
#pragma unroll
    for (int w = 0; w < COMPUTE_WARPS; ++w) {
      const float4 p = partial[(w * TILES + c.warp) * 32 + c.lane];
      sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
    }
  }
}

template <int MODE, typename OutT>
__global__ void __launch_bounds__(THREADS)
gemm_wide_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 OutT* __restrict__ out, int M, int N, int K, const Plan plan, int* __restrict__ error_flag) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], x_full;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kc = (K + BK - 1) / BK;
  const int stages = plan.stages, slot_bytes = plan.slot_bytes;
  const Phase phase{plan.tiles, plan.pieces, (kc + plan.pieces - 1) / plan.pieces, kc};
  unsigned char* x_s = smem;                       // kc pieces of [8 tokens x 64 k]
  unsigned char* ring = smem + (size_t)kc * (X_ROWS * 128);
  const int row0 = blockIdx.x * phase.tiles * 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], COMPUTE_WARPS);
    }
    mbar_init(&x_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dependency_launch();

  if (warp == COMPUTE_WARPS) {
    if (lane == 0) {
      // ---------------- copies
      const int total = phase.slots, ahead = total < stages ? total : stages;
      const int piece_bytes = phase.tiles * 16 * 128;
      bool ok = true;
      int g = 0, stage = 0;                        // the ring's next slot, and the parity of its barriers' phase
      unsigned parity = 0u;
      for (; g <= total; ++g) {
        if (g == ahead) {                          // weights first: nothing on the stream writes them
          grid_dependency_wait();                  // X comes from the kernel before this one
          mbar_expect_tx(&x_full, kc * (X_ROWS * 128));
          for (int i = 0; i < kc; ++i) tma_load_2d(x_s + (size_t)i * (X_ROWS * 128), &map_x, &x_full, i * BK, 0);
        }
        if (g == total) break;
        if (g >= stages && !(ok = mbar_wait(&empty_bar[stage], parity ^ 1u, error_flag, 1))) break;
        const int piece0 = g * phase.pieces, pieces = min(phase.pieces, kc - piece0);
        if (plan.bulk) {                           // one copy; pieces past the end arrive as zeros and count
          mbar_expect_tx(&full_bar[stage], phase.pieces * piece_bytes);
          tma_load_3d(ring + (size_t)stage * slot_bytes, &map_w, &full_bar[stage], 0, row0, piece0);
        } else {
          mbar_expect_tx(&full_bar[stage], pieces * piece_bytes);
          for (int j = 0; j < pieces; ++j)
            tma_load_2d(ring + (size_t)stage * slot_bytes + (size_t)j * piece_bytes, &map_w, &full_bar[stage],
                        (piece0 + j) * BK, row0);
        }
        if (++stage == stages) {
          stage = 0;
          parity ^= 1u;
        }
      }
      if (!ok || *reinterpret_cast<volatile int*>(error_flag) != 0) {
        // something gave up: let the copies still in flight land before the block may exit
        for (int j = g - 1; j >= 0 && j >= g - stages; --j) mbar_wait(&full_bar[j % stages], (j / stages) & 1, error_flag, 4);
        mbar_wait(&x_full, 0, error_flag, 4);
      }
    }
    // The other lanes of this warp do nothing, and must not wait for the predecessor here: a warp that
    // waits does so as a whole, and lane 0 would be held back from the loads above.
    return;
  }

  // ---------------- products
  grid_dependency_wait();
  Consumer c;
  c.full_bar = full_bar;
  c.empty_bar = empty_bar;
  c.stages = stages;
  c.slot_bytes = slot_bytes;
  c.ring_u32 = smem_u32(ring);
  c.warp = warp;
  c.lane = lane;
  c.group = warp >> 2;                             // the even or the odd pieces of a slot
  const int kk = warp & 3;                         // which 16 of a piece's 64 k
  c.a_offset = swizzled((lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4));
  c.b_offset = swizzled(lane & 7, 2 * kk + ((lane >> 3) & 1));
  c.error_flag = error_flag;
  c.stage = 0;
  c.parity = 0u;
  c.ok = mbar_wait(&x_full, 0, error_flag, 2);
  c.ok = __all_sync(0xffffffffu, c.ok);

  float4 sum;                                      // the ring is free when the sums meet: every slot has been read
  switch (phase.tiles) {
    case 1: product_tiles<1>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    case 2: product_tiles<2>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    case 3: product_tiles<3>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    case 4: product_tiles<4>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    case 5: product_tiles<5>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    case 6: product_tiles<6>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    case 7: product_tiles<7>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
    default: product_tiles<8>(c, phase, phase.slots, smem_u32(x_s), ring, sum); break;
  }
  if (c.ok && warp < phase.tiles) {
    // sum.x, sum.y: row (lane / 4) of the warp's tile, tokens 2 (lane % 4) and + 1;  sum.z, sum.w: the row eight further
    const int r = lane >> 2, t0 = 2 * (lane & 3);
    if (MODE == MODE_GATED) {
      const int feature = (blockIdx.x * phase.tiles + warp) * 8 + r, features = N / 2;
      if (feature < features) {
        if (t0 < M) out[(size_t)t0 * features + feature] = from_float<OutT>(silu_times(round_bf16(sum.x), round_bf16(sum.z)));
        if (t0 + 1 < M)
          out[(size_t)(t0 + 1) * features + feature] = from_float<OutT>(silu_times(round_bf16(sum.y), round_bf16(sum.w)));
      }
    } else {
      const int row = row0 + warp * 16 + r;
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
}

// How the product is laid out: 16-row tiles per block, pieces per slot, slots in the ring; false if it does
// not fit.  `budget` bounds the shared memory: what a block leaves free lets the next kernel's blocks start
// early, what it takes lets more of the weight be on its way before the predecessor has ended.
static bool plan_for(int N, int K, int budget, Plan* plan) {
  if (K <= 0 || N <= 0 || K % 8 != 0) return false;
  const long long kc = (K + BK - 1) / BK;
  const long long row_tiles = ((long long)N + 15) / 16;
  long long tiles = (row_tiles + multiprocessors() - 1) / multiprocessors();
  if (tiles > MAX_TILES) tiles = MAX_TILES;              // (more blocks than multiprocessors then)
  const long long piece_bytes = tiles * 16 * 128;
  long long pieces = SLOT_TARGET / piece_bytes;
  if (pieces < 2) pieces = 2;
  if (pieces > kc) pieces = kc;
  const long long slot = pieces * piece_bytes, slots = (kc + pieces - 1) / pieces;
  const long long x_bytes = kc * (X_ROWS * 128), partial = (long long)COMPUTE_WARPS * tiles * 512;
  long long stages = (budget - 1024 - x_bytes) / slot;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages > slots) stages = slots;
  if (stages < 2 && stages < slots) return false;
  long long ring = stages * slot;
  if (ring < partial) ring = partial;                    // the partial sums meet in the ring at the end
  if (x_bytes + ring + 1024 > SMEM_LIMIT) return false;
  plan->tiles = (int)tiles;
  plan->pieces = (int)pieces;
  plan->slot_bytes = (int)slot;
  plan->stages = (int)stages;
  plan->bulk = K % BK == 0;
  plan->smem = (int)(x_bytes + ring + 1024);
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

template <int MODE, typename OutT>
int launch(const void* X, const void* W, void* out, int M, int N, int K, int* error_flag, cudaStream_t stream) {
  Plan plan;
  MS_REQUIRE(plan_for(N, K, smem_budget(), &plan), "gemm_wide: an inner size of %d leaves no room for the weight ring", K);
  CUtensorMap map_w, map_x;
  const bool maps_ok = cached_map(&map_w, W, N, K, plan.tiles * 16, plan.bulk ? plan.pieces : 0) && cached_map(&map_x, X, M, K, X_ROWS);
  MS_REQUIRE(maps_ok, "gemm_wide: cuTensorMapEncodeTiled failed (M %d N %d K %d)", M, N, K);
  auto kernel = gemm_wide_kernel<MODE, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
    if (e != cudaSuccess) MS_FAIL("gemm_wide: cannot reserve shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int blocks = (int)(((long long)N + plan.tiles * 16 - 1) / (plan.tiles * 16));
  cudaError_t e = ms::launch(kernel, dim3(blocks), dim3(THREADS), (size_t)plan.smem, stream, map_w, map_x, (OutT*)out, M, N, K,
                             plan, error_flag);
  if (e != cudaSuccess) MS_FAIL("gemm_wide: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace wide
}  // namespace ms

using namespace ms;

// Whether ms_gemm_wide takes a product with this inner size (the activations and a ring of weight stages
// have to fit in shared memory): 0 no; 1 yes, with more blocks than multiprocessors; 2 yes, with at most one
// block per multiprocessor.
MS_EXPORT int ms_gemm_wide_supports(int N, int K) {
  wide::Plan plan;
  if (!wide::plan_for(N, K, wide::smem_budget(), &plan)) return 0;
  return ((long long)N + plan.tiles * 16 - 1) / (plan.tiles * 16) <= wide::multiprocessors() ? 2 : 1;
}

// X [M, K], W [N, K] bfloat16 (K a multiple of 8, both 16-byte aligned), M <= 8.
//   mode 0: out [M, N], bfloat16 (out_dtype 1) or float32 (0);
//   mode 1: W holds a gated feed-forward's gate and up projections in blocks of sixteen rows (eight gate rows,
//           then the up rows of the same eight features; N a multiple of 16); out [M, N / 2] bfloat16 =
//           silu(gate) * up.
// error_flag: one int on the device, zero before the first call; a kernel that gave up waiting writes a
// non-zero code there (1, 4 copies; 2, 3 products), which the caller checks when it synchronises.
MS_EXPORT int ms_gemm_wide(const void* X, const void* W, void* out, int out_dtype, int mode, int M, int N, int K,
                           int* error_flag, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  MS_REQUIRE(M <= wide::X_ROWS, "gemm_wide: %d rows; this kernel takes at most %d", M, wide::X_ROWS);
  MS_REQUIRE(K > 0 && K % 8 == 0, "gemm_wide: inner size %d is not a multiple of 8", K);
  MS_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_wide: operands must be 16-byte aligned");
  MS_REQUIRE(error_flag != nullptr, "gemm_wide: an error flag on the device is required");
  if (mode == wide::MODE_GATED) {
    MS_REQUIRE(N % 16 == 0 && out_dtype == MS_BF16, "gemm_wide: gated mode wants a multiple of 16 rows (%d) and bfloat16 results", N);
    return wide::launch<wide::MODE_GATED, __nv_bfloat16>(X, W, out, M, N, K, error_flag, stream);
  }
  MS_REQUIRE(mode == wide::MODE_PLAIN, "gemm_wide: unknown mode %d", mode);
  if (out_dtype == MS_BF16) return wide::launch<wide::MODE_PLAIN, __nv_bfloat16>(X, W, out, M, N, K, error_flag, stream);
  if (out_dtype == MS_F32) return wide::launch<wide::MODE_PLAIN, float>(X, W, out, M, N, K, error_flag, stream);
  MS_FAIL("gemm_wide: unknown output type code %d", out_dtype);
}
