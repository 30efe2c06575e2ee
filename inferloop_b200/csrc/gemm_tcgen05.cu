// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//     out[M,N] (+)= A[M,K] * W[N,K]^T (+ bias[N]),  32-bit accumulation in tensor memory,
// or, for a weight whose rows interleave 64 gate rows with their 64 up rows,
//     out[M,N/2] = silu(gate) * up   (the SwiGLU product in the epilogue).
//
// One kernel serves decode-shaped (few tokens) and prefill-shaped (many tokens) products.
// tcgen05.mma computes D[128 x BN] = X[128 x K] * Y[BN x K]^T with both operands K-major in
// shared memory.  With few tokens the operands are swapped: X is a 128-row tile of the
// WEIGHT and Y the (padded) tokens, so every tensor-core row does useful work and the
// kernel is a pure stream of weight tiles; with many tokens X is a 128-token tile and Y a
// tile of BN weight rows.
//
// Per CTA (192 threads, 320 with two row blocks per tile):
//   warp 0      one lane issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle,
//               no cluster multicast) into a ring of STAGES buffers; the first ring of WEIGHT
//               tiles is requested before tensor memory is allocated and before the kernel
//               waits for its predecessor (the weights depend on neither);
//   warp 1      allocates tensor memory (two accumulators); one lane issues tcgen05.mma
//               (4 per 64-wide K block) and tcgen05.commit to hand buffers back and to
//               signal that an accumulator is complete;
//   warps 2-5   read an accumulator with tcgen05.ld and write the result while the next
//               tile accumulates in the other one.
// How the work is dealt out (host side, end of this file):
//   few tokens, tiles <= 2 CTAs per SM: every tile's K range is cut into 1, 2, 4 or 8 equal
//     parts, one per CTA of a thread-block cluster.  Each CTA SENDS the rows of its share to
//     the CTA that owns them (st.async, counted by the owner's mbarrier); the owner adds the
//     shares in K order from its own shared memory and writes out (token tiles up to 64; the
//     128-token tile keeps the older form in which owners read their peers' shares between
//     two cluster barriers).  One cluster barrier, at the start.
//     Accumulating products of up to eight tokens with a large weight skip the cluster: the K
//     ranges are separate CTAs that add their shares into the 32-bit output (red.add.v4).
//   few tokens, many tiles (the output matrix): a persistent grid takes equal, contiguous runs
//     of (tile, K block) units ("stream-K"); a tile shared by two CTAs goes through a 32-bit
//     workspace slot and a ticket: the CTA that takes the tile's last ticket adds the shares in
//     K order, so the sum does not depend on which CTA finished first.
//   many tokens: whole tiles in rounds of equal size, all CTAs of a round starting at K block
//     0 together so that they share operand blocks in L2; with few tiles, equal K ranges per
//     tile (a cluster that shares the write-out by columns, or tickets for two-block tiles).
//   many tokens and enough 256 x 256 tiles: `gemm_pair_kernel` further down, a cluster of two
//     CTAs per tile that the tensor cores treat as one unit (tcgen05.mma.cta_group::2), each
//     CTA loading its own half of the weight block.
// There is no spin-wait on another CTA anywhere.  Decode-shaped launches keep their ring below
// half of an SM's shared memory: two CTAs per SM.  Every mbarrier wait is bounded: on expiry the
// kernel raises a flag in global memory, drains what it armed, frees its tensor memory and returns.
//
// The reference computes these products with JIT-compiled tile kernels that target no
// architecture in particular, or with cuBLAS (crates/backend/cuda-kernels/src/tile/
// projection/prefill_gemm_kernels.rs:11-69, small_gemm_kernels.rs:10-29;
// crates/backend/cuda/src/device/cublaslt.rs:38-42).
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

namespace {

constexpr int kBlockK = 64;            // bf16 elements per K block = one 128-byte swizzle row
constexpr int kTileX = 128;            // rows of the X operand = MMA M
constexpr int threads_for(int ms) { return 64 + 128 * ms; }   // TMA warp, MMA warp, four epilogue warps per 128 rows

enum Epilogue : int { kStore = 0, kAccumulate = 1, kSwiGLU = 2 };

// silu(g) * u with the fast reciprocal: the quotient is within 2 ulp, far inside what the
// bfloat16 result keeps, and an epilogue thread has 128 of these per tile.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row
// groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// D = 32-bit, A and B = bfloat16, both K-major, N and M encoded.
__host__ __device__ constexpr uint32_t instr_desc(int mma_m, int mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(mma_n >> 3) << 17) | ((uint32_t)(mma_m >> 4) << 24);
}

struct Params {
  void* out;                 // [M, N], bf16 or f32
  const float* bias;         // [N] or null
  float* partial;            // stream-K workspace: two slots of [BN][128] floats per CTA
  int* tickets;              // one counter per tile, zero between launches
  int* error_flag;           // set to 1 when a bounded wait ran out
  int M, N, K, ldo;
  int tiles_x, tiles_y;      // tiles of the X operand (128 rows) and of the Y operand (BN rows)
  int k_blocks;              // ceil(K / 64)
  long long units;           // K blocks of the tiles that are shared out stream-K fashion
  int sk_ctas;               // CTAs that share them (0: all of the grid, or one per unit if those are fewer)
  int dp_waves;              // whole-tile rounds before that: CTA c takes tiles c, c + grid, ...
  long long sk_tile0;        // tiles of those rounds (the last round may be short) = first tile of the stream-K part
  int epilogue;              // Epilogue
  int out_f32;               // element type of out
  int cluster;               // > 1: a tile's K ranges belong to the CTAs of one cluster, added through their shared memory
  int tma_out;               // many tokens: the result leaves through shared memory and TMA stores (adds, when accumulating)
  int red_out;               // few tokens, accumulating: the K ranges of a tile are separate CTAs whose shares meet in memory (red.add)
};

// Work: first `dp_waves` rounds of WHOLE tiles in wave order (round w: CTA c takes tile
// w * grid + c, so the CTAs of a round work on neighbouring tiles and share operand tiles
// in L2), then the remaining tiles stream-K fashion: a unit is one 64-wide K block of one
// of those tiles and the CTAs take equal, contiguous runs of units, so a CTA handles the
// tail of one tile, some whole tiles, and the head of another.  `units`, `start`, `cta_of`
// and `slot` speak of the stream-K part only.
struct Schedule {
  long long units; int grid, k_blocks;
  __device__ __forceinline__ long long start(int c) const { return (long long)c * units / grid; }
  __device__ __forceinline__ int cta_of(long long u) const { return (int)(((u + 1) * grid - 1) / units); }
  // slot of CTA c's contribution to the tile whose first unit is `tile_first`
  __device__ __forceinline__ int slot(int c, long long tile_first) const { return 2 * c + (start(c) >= tile_first ? 0 : 1); }
};

// The segments (tile, first K block, number of K blocks) of one CTA, in order.
struct Segments {
  int w, dp_waves, grid, cta, k_blocks;
  long long u, u_end, sk_tile0;
  __device__ Segments(const Params& p, const Schedule& sch, int cta_, int grid_)
      : w(0), dp_waves(p.dp_waves), grid(grid_), cta(cta_), k_blocks(p.k_blocks),
        u(0), u_end(0), sk_tile0(p.sk_tile0) {
    if (p.units > 0 && cta_ < sch.grid) { u = sch.start(cta_); u_end = sch.start(cta_ + 1); }
  }
  // sk_first: first stream-K unit of the tile, or -1 for a whole tile of the wave part
  __device__ __forceinline__ bool next(long long& tile, int& kb0, int& cnt, long long& sk_first) {
    if (w < dp_waves) {
      tile = (long long)w * grid + cta; kb0 = 0; cnt = k_blocks; sk_first = -1; ++w;
      if (tile < sk_tile0) return true;
      w = dp_waves;                                 // the last round has no tile for this CTA
    }
    if (u >= u_end) return false;
    const long long t = u / k_blocks;
    tile = sk_tile0 + t; kb0 = (int)(u % k_blocks);
    cnt = (int)min((long long)(k_blocks - kb0), u_end - u);
    sk_first = t * k_blocks;
    u += cnt;
    return true;
  }
};

// MS = 128-row blocks of the X operand per tile.  MS = 1: one accumulator per tile, two of
// them in tensor memory, so a tile is written out while the next accumulates.  MS = 2 (many
// tokens): a tile is 256 x BN, its two halves share every Y block that comes in, which cuts
// the bytes per flop that L2 has to deliver by a third; both accumulators belong to the
// tile, and eight epilogue warps drain them together.
template <int BN, int STAGES, bool SWAP, int MS>
__global__ void __launch_bounds__(threads_for(MS), SWAP ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
               const __grid_constant__ CUtensorMap map_out, const Params p) {
  static_assert(MS == 1 || (MS == 2 && !SWAP), "two row blocks per tile only for the many-token form");
  constexpr uint32_t kBytesX1 = kTileX * kBlockK * 2;          // one 128-row block of X
  constexpr uint32_t kBytesX = MS * kBytesX1;
  constexpr uint32_t kBytesY = BN * kBlockK * 2;
  constexpr uint32_t kStageBytes = kBytesX + kBytesY;          // multiples of 1024
  constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;             // columns of one accumulator
  constexpr uint32_t kTmemCols = 2 * kAccCols <= 64 ? 64 : 2 * kAccCols <= 128 ? 128 : 2 * kAccCols <= 256 ? 256 : 512;   // two accumulators; a power of two
  constexpr int kTileFloats = BN * kTileX;                     // one 128-row block of a tile
  constexpr int kBufs = MS == 1 ? 2 : 1;                       // tiles that tensor memory holds
  constexpr int kEpiThreads = 128 * MS;
  // Few tokens and a cluster: every CTA SENDS the rows of its share to the CTA that owns them
  // (asynchronous stores that count on the owner's mbarrier), so the owner waits for bytes,
  // not for the whole cluster, and nobody reads a peer's memory.  Wider token tiles keep the
  // form in which the owner fetches the shares.
  constexpr bool kPush = SWAP && BN <= 64;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only 16-byte aligned by contract; align by hand
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  // many tokens: one 128-row x 128-byte block per row block of the tile, where results are laid
  // out (128-byte swizzle) for the TMA store that takes them to memory
  constexpr uint32_t kStagingBytes = SWAP ? 0u : (uint32_t)MS * kTileX * 128u;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes + kStagingBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
  const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* flags = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 5);   // [0] = failed, [1] = last ticket
  const uint32_t red_bar = smem_u32(bars + 2 * STAGES + 6);                        // counts the bytes of the shares sent here
  // [32][64] SwiGLU exchange of whole tiles (swap mode), or the shares sent by the cluster:
  // [source CTA][gate, up][BN / 4][rows of this CTA][4]
  float* xch = reinterpret_cast<float*>(bars + 2 * STAGES + 8);
  const bool push = kPush && p.cluster > 1;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The stream-K part is shared by the first min(grid, units) CTAs, so that every CTA that
  // takes part holds at least one unit (a tile's sharers are then consecutive CTAs).
  const int sk_grid = p.sk_ctas > 0 ? p.sk_ctas : p.units < (long long)gridDim.x ? (int)p.units : (int)gridDim.x;
  const Schedule sch{p.units > 0 ? p.units : 1, sk_grid > 0 ? sk_grid : 1, p.k_blocks};
  const bool in_sk = p.units > 0 && (int)blockIdx.x < sk_grid;
  const long long u_begin = in_sk ? sch.start(blockIdx.x) : 0, u_end = in_sk ? sch.start(blockIdx.x + 1) : 0;

  // The units of this CTA in order, one K block a step; the divisions that find a tile's
  // place happen once per segment, not per block: the producer lane's issue rate bounds the ring.
  struct Units {
    Segments segs;
    int tiles_x, kb, left, x0, y0;
    __device__ Units(const Params& p, const Schedule& sch) : segs(p, sch, blockIdx.x, gridDim.x), tiles_x(p.tiles_x), kb(0), left(0), x0(0), y0(0) {}
    __device__ __forceinline__ bool next(int& kcol, int& x, int& y) {
      if (left == 0) {
        long long tile, sk_first;
        int kb0, cnt;
        if (!segs.next(tile, kb0, cnt, sk_first)) return false;
        kb = kb0; left = cnt;
        x0 = (int)(tile % tiles_x) * (MS * kTileX);
        y0 = (int)(tile / tiles_x) * BN;
      }
      kcol = kb * kBlockK; x = x0; y = y0;
      ++kb; --left;
      return true;
    }
  };
  auto load_x = [&](uint32_t dst, uint32_t bar, int kcol, int x0) {
#pragma unroll
    for (int ms = 0; ms < MS; ++ms) tma_load_2d(dst + ms * kBytesX1, &map_x, bar, kcol, x0 + ms * kTileX);
  };
  uint32_t n_units = 0, n_early = 0;            // of the producer lane (thread 0)
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, kEpiThreads); }
    if (push) mbar_init(red_bar, 1);
    flags[0] = 0; flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (push) mbar_expect_tx(red_bar, (uint32_t)(kTileX * BN * 4));   // one whole tile's worth of rows arrives here
    // The weight operand depends on no earlier kernel and on no other thread of this CTA:
    // the first ring of weight tiles is requested right here, before tensor memory is
    // allocated and before this kernel waits for its predecessor; the activation tiles of
    // those stages follow the wait.
    long long my_tiles = (long long)blockIdx.x < p.sk_tile0 ? (p.sk_tile0 - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    if (my_tiles > p.dp_waves) my_tiles = p.dp_waves;
    const uint32_t n_dp = (uint32_t)my_tiles * (uint32_t)p.k_blocks;
    n_units = n_dp + (uint32_t)(u_end - u_begin);
    n_early = n_units < (uint32_t)STAGES ? n_units : (uint32_t)STAGES;
    Units early(p, sch);
    for (uint32_t it = 0; it < n_early; ++it) {
      int kcol, x0, y0;
      early.next(kcol, x0, y0);
      const uint32_t dst = base + it * kStageBytes;
      mbar_expect_tx(full0 + 8 * it, kStageBytes);
      if (SWAP) load_x(dst, full0 + 8 * it, kcol, x0);
      else tma_load_2d(dst + kBytesX, &map_y, full0 + 8 * it, kcol, y0);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  if (push) cluster_sync_all();          // every peer's mbarrier is ready before anything is sent to it
  else __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      pdl_wait();
      Units units(p, sch);
      for (uint32_t it = 0; it < n_early; ++it) {
        int kcol, x0, y0;
        units.next(kcol, x0, y0);
        const uint32_t dst = base + it * kStageBytes;
        if (SWAP) tma_load_2d(dst + kBytesX, &map_y, full0 + 8 * it, kcol, y0);
        else load_x(dst, full0 + 8 * it, kcol, x0);
      }
      for (uint32_t it = n_early; it < n_units; ++it) {
        const uint32_t s = it % STAGES;
        ok = mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1);
        if (!ok) break;
        int kcol, x0, y0;
        if (!units.next(kcol, x0, y0)) break;
        const uint32_t dst = base + s * kStageBytes;
        mbar_expect_tx(full0 + 8 * s, kStageBytes);
        load_x(dst, full0 + 8 * s, kcol, x0);
        tma_load_2d(dst + kBytesX, &map_y, full0 + 8 * s, kcol, y0);
      }
      if (!ok) { flags[0] = 1; if (p.error_flag) *p.error_flag = 1; }
    }
    if (!SWAP && p.cluster > 1) { cluster_sync_all(); cluster_sync_all(); }   // the epilogue warps meet the cluster twice; so must every thread
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(kTileX, BN);
      bool ok = true;
      uint32_t it = 0, seg = 0;
      Segments segs(p, sch, blockIdx.x, gridDim.x);
      long long tile_, sk_first_;
      int kb0, cnt;
      for (; ok && segs.next(tile_, kb0, cnt, sk_first_); ++seg) {
        const uint32_t b = seg % kBufs;
        ok = mbar_wait(tempty0 + 8 * b, ((seg / kBufs) & 1) ^ 1);  // the epilogue has drained this accumulator
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t acc = tmem_base + (MS == 1 ? b * kAccCols : 0u);
        for (int i = 0; i < cnt; ++i, ++it) {
          const uint32_t s = it % STAGES;
          ok = mbar_wait(full0 + 8 * s, (it / STAGES) & 1);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a = base + s * kStageBytes;
          const uint64_t db = smem_desc(a + kBytesX);
#pragma unroll
          for (int ms = 0; ms < MS; ++ms) {
            const uint64_t da = smem_desc(a + ms * kBytesX1);
#pragma unroll
            for (int k = 0; k < kBlockK / 16; ++k)
              mma_bf16(acc + ms * kAccCols, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(empty0 + 8 * s);       // the buffer is free once these MMAs have read it
        }
        tcgen05_commit(tfull0 + 8 * b);         // arrives when every MMA issued so far is complete
      }
      if (!ok) {
        flags[0] = 1; if (p.error_flag) *p.error_flag = 1;
        tcgen05_commit(tfull0); tcgen05_commit(tfull0 + 8);       // let the epilogue leave its wait
      }
    }
    if (!SWAP && p.cluster > 1) { cluster_sync_all(); cluster_sync_all(); }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5, and 6..9 for the second row block)
    pdl_wait();                               // outputs, shares and tickets belong to earlier kernels until now
    const int quad = warp & 3;                // tensor-memory lanes 32*quad .. 32*quad+31
    const int ms = (warp - 2) >> 2;           // row block of the tile
    const int row = quad * 32 + lane;         // row of that block this thread owns
    constexpr int CH = BN < 32 ? BN : 32;     // columns per tensor-memory read
    uint32_t seg = 0;
    bool failed = false;
    bool met_cluster = false;                 // many-token form with a cluster: every thread meets it exactly once
    Segments segs(p, sch, blockIdx.x, gridDim.x);
    long long tile, tile_first;
    int kb0, cnt;
    for (; !failed && segs.next(tile, kb0, cnt, tile_first); ++seg) {
      const int x0 = (int)(tile % p.tiles_x) * (MS * kTileX) + ms * kTileX, y0 = (int)(tile / p.tiles_x) * BN;
      const int xr = x0 + row;
      const uint32_t b = seg % kBufs;
      if (!mbar_wait(tfull0 + 8 * b, (seg / kBufs) & 1)) { flags[0] = 1; if (p.error_flag) *p.error_flag = 1; }
      tcgen05_fence_after();
      failed = flags[0] != 0;
      if (failed) break;
      int col_lo = 0, col_hi = BN;             // columns this CTA writes out
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (MS == 1 ? b : (uint32_t)ms) * kAccCols;
      // Many tokens, accumulating into the 32-bit output through TMA: the write-out ADDS in
      // memory, so a K range of a tile is written out like a whole tile and the ranges of a
      // tile meet in memory (in whatever order they finish: a 32-bit sum of the same terms).
      const bool additive = !SWAP && p.tma_out && p.epilogue == kAccumulate && p.cluster == 1;
      const bool whole = cnt == p.k_blocks || additive;
      const bool with_bias = p.bias != nullptr && (kb0 == 0 || !additive);   // once per output: of the ranges that meet in memory, the first adds it
      bool last = whole;
      int c_first = 0, c_last = 0;
      if (SWAP && !whole && p.red_out) {
        // Few tokens, accumulating into the 32-bit output: this CTA's K range is added in
        // memory, where the other ranges of the tile meet it (a 32-bit sum of the same terms
        // in whatever order they arrive); no cluster, nothing exchanged, nothing waited for.
        // The share goes through shared memory ([token][row]; the stage ring is idle, every load
        // into it has been consumed) so that a thread adds four neighbouring features at once.
        float* red = reinterpret_cast<float*>(smem);
        const float bv = (p.bias && kb0 == 0 && xr < p.N) ? p.bias[xr] : 0.f;
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          if (CH == 32) tmem_load_32(taddr + c0, v); else tmem_load_16(taddr + c0, v);
#pragma unroll
          for (int c = 0; c < CH; ++c) red[(c0 + c) * kTileX + row] = v[c] + bv;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool vec = (p.ldo % 4 == 0) && ((uintptr_t)p.out % 16 == 0) && (x0 + kTileX <= p.N);
        for (int q = (int)threadIdx.x - 64; q < BN * (kTileX / 4); q += 128) {
          const int c = q / (kTileX / 4), r4 = (q % (kTileX / 4)) * 4;
          const int m = y0 + c;
          if (m >= p.M) break;
          const float4 val = *reinterpret_cast<const float4*>(red + c * kTileX + r4);
          float* dst = (float*)p.out + (size_t)m * p.ldo + x0 + r4;
          if (vec) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(val.x), "f"(val.y), "f"(val.z), "f"(val.w) : "memory");
          } else {
            const float e[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (x0 + r4 + j < p.N) atomicAdd(dst + j, e[j]);
          }
        }
        break;
      }
      if (kPush && !whole && p.cluster > 1) {
        // The S CTAs of a cluster hold the S consecutive K ranges of one tile.  CTA r owns 1/S
        // of the tile's rows (of its gate rows and their up rows): every CTA sends the rows of
        // its share to their owners, [source][gate, up][column / 4][row][4].
        const int S = p.cluster;
        const bool sw = p.epilogue == kSwiGLU;
        const int parts = sw ? 2 : 1;
        const int rows_per = (sw ? 64 : kTileX) / S;
        const int rr = sw ? (row & 63) : row;
        const uint32_t owner = (uint32_t)(rr / rows_per);
        const int rl = rr % rows_per, part = sw ? (row >> 6) : 0;
        const uint32_t me = cluster_rank();
        const uint32_t dst0 = peer_addr(smem_u32(xch) + 16u * (uint32_t)(((int)me * parts + part) * (BN / 4) * rows_per + rl), owner);
        const uint32_t bar = peer_addr(red_bar, owner);
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          if (CH == 32) tmem_load_32(taddr + c0, v); else tmem_load_16(taddr + c0, v);
#pragma unroll
          for (int g = 0; g < CH / 4; ++g)
            st_peer_v4(dst0 + 16u * (uint32_t)((c0 / 4 + g) * rows_per), bar, v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
        // ... and adds, in the order of increasing K, the shares of the rows it owns.
        const int r = (int)me;
        const int t = (int)threadIdx.x - 64;
        const int my_rl = t % rows_per;
        const int my_row = r * rows_per + my_rl;
        const int n = sw ? (x0 / kTileX) * 64 + my_row : x0 + my_row;       // output feature
        const int n_end = sw ? p.N / 2 : p.N;
        const float bv = (p.bias && n < n_end) ? p.bias[n] : 0.f;
        bool arrived = false;
        for (int cg = t / rows_per; cg < BN / 4; cg += 128 / rows_per) {
          float old[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = y0 + cg * 4 + j;
            old[j] = (p.epilogue == kAccumulate && m < p.M && n < n_end) ? __ldcg((const float*)p.out + (size_t)m * p.ldo + n) : 0.f;
          }
          if (!arrived) {
            if (!mbar_wait(red_bar, 0)) { flags[0] = 1; if (p.error_flag) *p.error_flag = 1; break; }
            arrived = true;
          }
          float acc[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
          const float4* slots = reinterpret_cast<const float4*>(xch);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (q < S) {
              const float4 a = slots[((q * parts) * (BN / 4) + cg) * rows_per + my_rl];
              acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
              if (sw) {
                const float4 u = slots[((q * parts + 1) * (BN / 4) + cg) * rows_per + my_rl];
                up[0] += u.x; up[1] += u.y; up[2] += u.z; up[3] += u.w;
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = y0 + cg * 4 + j;
            if (m < p.M && n < n_end) {
              const float val = sw ? silu_mul(acc[j], up[j]) : acc[j] + bv + old[j];
              const size_t o = (size_t)m * p.ldo + n;
              if (p.out_f32) ((float*)p.out)[o] = val; else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(val);
            }
          }
        }
        // a thread without rows of its own still stays until the shares sent here have landed
        if (!arrived && !mbar_wait(red_bar, 0)) { flags[0] = 1; if (p.error_flag) *p.error_flag = 1; }
        break;
      }
      if (SWAP && !whole && p.cluster > 1) {
        // This CTA's share goes to its own shared memory ([col][row]; the stage ring is idle,
        // every load into it has been consumed); the cluster adds the shares after the roles.
        float* red = reinterpret_cast<float*>(smem);
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          if (CH == 32) tmem_load_32(taddr + c0, v); else tmem_load_16(taddr + c0, v);
#pragma unroll
          for (int c = 0; c < CH; ++c) red[(c0 + c) * kTileX + row] = v[c];
        }
        break;
      }
      const bool peers = !SWAP && !whole && p.cluster > 1;     // many tokens, a tile's K ranges over a cluster
      if (peers) {
        // The sharers of this tile are the CTAs of this cluster.  Each parks its share in its
        // own shared memory ([col][row]; the stage ring is idle, every load into it has been
        // consumed); after the barrier every CTA adds the shares of ITS columns, in K order,
        // straight from its peers' shared memory, and writes them out.
        float* red = reinterpret_cast<float*>(smem);
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          if (CH == 32) tmem_load_32(taddr + c0, v); else tmem_load_16(taddr + c0, v);
#pragma unroll
          for (int c = 0; c < CH; ++c) red[(c0 + c) * kTileX + row] = v[c];
        }
        cluster_sync_all();
        met_cluster = true;
        const int per = BN / p.cluster;
        col_lo = (int)cluster_rank() * per;
        col_hi = col_lo + per;
        last = true;
      } else if (!whole) {
        // 1. park this CTA's share of the tile: [col][row], a warp writes 128 contiguous bytes
        float* mine = p.partial + ((size_t)sch.slot(blockIdx.x, tile_first) * MS + ms) * kTileFloats;
        for (int c0 = 0; c0 < BN; c0 += CH) {
          float v[32];
          if (CH == 32) tmem_load_32(taddr + c0, v); else tmem_load_16(taddr + c0, v);
#pragma unroll
          for (int c = 0; c < CH; ++c) mine[(size_t)(c0 + c) * kTileX + row] = v[c];
        }
        tcgen05_fence_before();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tempty0 + 8 * b) : "memory");
        c_first = sch.cta_of(tile_first);
        c_last = sch.cta_of(tile_first + p.k_blocks - 1);
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (threadIdx.x == 64) {
          const int t = atomicAdd(p.tickets + tile, 1);
          const int n = c_last - c_first + 1;
          flags[1] = (t == n - 1) ? 1 : 0;
          if (t == n - 1) p.tickets[tile] = 0;               // ready for the next launch
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        last = flags[1] != 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");        // flags[1] is reused by the next segment
        if (last) __threadfence();
      }
      if (last) {
        // values of columns c0 .. c0 + CH of this thread's row: from the accumulator, or the
        // tile's shares added in the fixed order of increasing K
        auto fetch = [&](int c0, float (&v)[32]) {
          if (whole) {
            if (CH == 32) tmem_load_32(taddr + c0, v); else tmem_load_16(taddr + c0, v);
          } else if (peers) {
#pragma unroll
            for (int c = 0; c < CH; ++c) v[c] = 0.f;
            for (int q0 = 0; q0 < p.cluster; q0 += 2) {        // two peers' loads in flight together
              float a[2][CH];
#pragma unroll
              for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < CH; ++c)
                  a[j][c] = q0 + j < p.cluster ? ld_peer_f32(base + (uint32_t)((c0 + c) * kTileX + row) * 4u, (uint32_t)(q0 + j)) : 0.f;
#pragma unroll
              for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < CH; ++c) v[c] += a[j][c];
            }
          } else {
#pragma unroll
            for (int c = 0; c < CH; ++c) v[c] = 0.f;
            // shares are fetched kBatch CTAs at a time so that their loads are all in flight
            constexpr int kBatch = CH == 16 ? 4 : 2;
            for (int cc = c_first; cc <= c_last; cc += kBatch) {
              float a[kBatch][CH];
#pragma unroll
              for (int j = 0; j < kBatch; ++j) {
                const bool on = cc + j <= c_last;
                const float* src = p.partial + ((size_t)sch.slot(on ? cc + j : cc, tile_first) * MS + ms) * kTileFloats + row;
#pragma unroll
                for (int c = 0; c < CH; ++c) a[j][c] = on ? __ldcg(src + (size_t)(c0 + c) * kTileX) : 0.f;
              }
#pragma unroll
              for (int j = 0; j < kBatch; ++j)
#pragma unroll
                for (int c = 0; c < CH; ++c) v[c] += a[j][c];
            }
          }
        };
        if (!SWAP && p.tma_out) {
          // A thread's 128 bytes of one output row go to the staging block (row = its tile row,
          // 16-byte pieces swizzled as the tensor map says); one thread of the row block then
          // hands the block to TMA, which writes whole lines, clips what lies outside the
          // matrix and, when accumulating, adds in memory instead of storing.
          const uint32_t stg = base + STAGES * kStageBytes + (uint32_t)ms * (kTileX * 128u);
          const bool elected = row == 0;
          auto group_sync = [&]() {                          // the 128 threads of this row block
            if (ms == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
            else asm volatile("bar.sync 3, 128;" ::: "memory");
          };
          auto flush_row = [&](const uint4 (&piece)[8], int out_col) {
            if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // the block's last reader is done
            group_sync();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (uint32_t)row * 128u + (uint32_t)((j ^ (row & 7)) << 4)),
                           "r"(piece[j].x), "r"(piece[j].y), "r"(piece[j].z), "r"(piece[j].w) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            group_sync();
            if (elected) {
              if (p.epilogue == kAccumulate)
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                             ::"l"(&map_out), "r"(stg), "r"(out_col), "r"(x0) : "memory");
              else
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                             ::"l"(&map_out), "r"(stg), "r"(out_col), "r"(x0) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          };
          auto pack8 = [&](const float* r8) {                // eight floats as bf16 in 16 bytes
            uint4 q;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(r8[0], r8[1]), h1 = __floats2bfloat162_rn(r8[2], r8[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(r8[4], r8[5]), h3 = __floats2bfloat162_rn(r8[6], r8[7]);
            q.x = *reinterpret_cast<uint32_t*>(&h0); q.y = *reinterpret_cast<uint32_t*>(&h1);
            q.z = *reinterpret_cast<uint32_t*>(&h2); q.w = *reinterpret_cast<uint32_t*>(&h3);
            return q;
          };
          uint4 piece[8];
          if (p.epilogue == kSwiGLU) {
            // columns come in blocks of 64 gate then 64 up: 64 outputs = one 128-byte row of bf16
            for (int cb = col_lo; cb < col_hi; cb += 128) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                float g[32], u[32], r[32];
                fetch(cb + 32 * half, g);
                fetch(cb + 64 + 32 * half, u);
#pragma unroll
                for (int c = 0; c < 32; ++c) r[c] = silu_mul(g[c], u[c]);
#pragma unroll
                for (int j = 0; j < 4; ++j) piece[4 * half + j] = pack8(r + 8 * j);
              }
              flush_row(piece, (y0 + cb) / 2);
            }
          } else if (p.out_f32) {
            for (int c0 = col_lo; c0 < col_hi; c0 += 32) {
              float v[32];
              fetch(c0, v);
              if (with_bias) {
#pragma unroll
                for (int c = 0; c < 32; ++c) v[c] += (y0 + c0 + c < p.N) ? p.bias[y0 + c0 + c] : 0.f;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j)
                piece[j] = make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
              flush_row(piece, y0 + c0);
            }
          } else {
            for (int c0 = col_lo; c0 < col_hi; c0 += 64) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                float v[32];
                fetch(c0 + 32 * half, v);
                if (p.bias) {
#pragma unroll
                  for (int c = 0; c < 32; ++c) v[c] += (y0 + c0 + 32 * half + c < p.N) ? p.bias[y0 + c0 + 32 * half + c] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) piece[4 * half + j] = pack8(v + 8 * j);
              }
              flush_row(piece, y0 + c0);
            }
          }
        } else
        if (p.epilogue == kSwiGLU) {
          // The weight rows come in blocks of 64 gate rows followed by their 64 up rows; the
          // output has half as many features: out[m, i] = silu(gate_i) * up_i.
          const int half_n = p.N / 2;
          if (SWAP) {
            // gate rows are tile rows 0..63, up rows 64..127: the up half hands its values to
            // the gate half through shared memory
            const int i = (x0 / kTileX) * 64 + (row & 63);
            for (int c0 = 0; c0 < BN; c0 += CH) {
              float v[32];
              fetch(c0, v);
              if (row >= 64) {
#pragma unroll
                for (int c = 0; c < CH; ++c) xch[c * 64 + (row - 64)] = v[c];
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (row < 64 && i < half_n) {
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                  const int m = y0 + c0 + c;
                  if (m < p.M) {
                    const float g = v[c], u = xch[c * 64 + row];
                    const float r = silu_mul(g, u);
                    const size_t o = (size_t)m * p.ldo + i;
                    if (p.out_f32) ((float*)p.out)[o] = r; else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(r);
                  }
                }
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
            }
          } else {
            // columns come in blocks of 64 gate then 64 up; a thread holds both halves
            for (int cb = col_lo; cb < col_hi; cb += 128) {
              for (int c0 = cb; c0 < cb + 64; c0 += CH) {
                float g[32], u[32];
                fetch(c0, g);
                fetch(c0 + 64, u);
                const int i0 = (y0 + cb) / 2 + (c0 - cb);
                float r[32];
#pragma unroll
                for (int c = 0; c < CH; ++c) r[c] = silu_mul(g[c], u[c]);
                if (xr < p.M) {
                  const size_t o = (size_t)xr * p.ldo + i0;
                  const bool full = i0 + CH <= half_n && (p.ldo % 8 == 0) && ((uintptr_t)p.out % 16 == 0) && !p.out_f32;
                  if (full) {
                    uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + o);
#pragma unroll
                    for (int c = 0; c < CH / 8; ++c) {
                      uint4 q;
                      __nv_bfloat162 h0 = __floats2bfloat162_rn(r[8 * c], r[8 * c + 1]);
                      __nv_bfloat162 h1 = __floats2bfloat162_rn(r[8 * c + 2], r[8 * c + 3]);
                      __nv_bfloat162 h2 = __floats2bfloat162_rn(r[8 * c + 4], r[8 * c + 5]);
                      __nv_bfloat162 h3 = __floats2bfloat162_rn(r[8 * c + 6], r[8 * c + 7]);
                      q.x = *reinterpret_cast<uint32_t*>(&h0); q.y = *reinterpret_cast<uint32_t*>(&h1);
                      q.z = *reinterpret_cast<uint32_t*>(&h2); q.w = *reinterpret_cast<uint32_t*>(&h3);
                      dst[c] = q;
                    }
                  } else {
#pragma unroll
                    for (int c = 0; c < CH; ++c) {
                      if (i0 + c < half_n) {
                        if (p.out_f32) ((float*)p.out)[o + c] = r[c]; else ((__nv_bfloat16*)p.out)[o + c] = __float2bfloat16_rn(r[c]);
                      }
                    }
                  }
                }
              }
            }
          }
        } else
        for (int c0 = col_lo; c0 < col_hi; c0 += CH) {
          float v[32];
          fetch(c0, v);
          if (SWAP) {
            // X rows are output features n = xr; columns are tokens m = y0 + c
            if (xr < p.N) {
              const float bv = p.bias ? p.bias[xr] : 0.f;
              if (p.epilogue == kAccumulate) {
                // all the old values first: the loads are in flight together
                float old[CH];
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                  const int m = y0 + c0 + c;
                  old[c] = m < p.M ? __ldcg((const float*)p.out + (size_t)m * p.ldo + xr) : 0.f;
                }
#pragma unroll
                for (int c = 0; c < CH; ++c) v[c] += old[c];
              }
#pragma unroll
              for (int c = 0; c < CH; ++c) {
                const int m = y0 + c0 + c;
                if (m < p.M) {
                  const size_t o = (size_t)m * p.ldo + xr;
                  const float r = v[c] + bv;
                  if (p.out_f32) ((float*)p.out)[o] = r;
                  else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(r);
                }
              }
            }
          } else {
            // X rows are tokens m = xr; columns are output features n = y0 + c
            const int n0 = y0 + c0;
            const bool full = n0 + CH <= p.N && (p.ldo % 8 == 0) && ((uintptr_t)p.out % 16 == 0);
            if (xr < p.M && full) {
              // a whole chunk of this row: 16-byte accesses
              const size_t o = (size_t)xr * p.ldo + n0;
              if (p.bias) {
#pragma unroll
                for (int c = 0; c < CH; ++c) v[c] += p.bias[n0 + c];
              }
              if (p.out_f32) {
                float4* dst = reinterpret_cast<float4*>((float*)p.out + o);
#pragma unroll
                for (int c = 0; c < CH / 4; ++c) {
                  float4 r = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                  if (p.epilogue == kAccumulate) {
                    const float4 old = dst[c];
                    r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
                  }
                  dst[c] = r;
                }
              } else {
                uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)p.out + o);
#pragma unroll
                for (int c = 0; c < CH / 8; ++c) {
                  uint4 r;
                  __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * c], v[8 * c + 1]);
                  __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * c + 2], v[8 * c + 3]);
                  __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * c + 4], v[8 * c + 5]);
                  __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * c + 6], v[8 * c + 7]);
                  r.x = *reinterpret_cast<uint32_t*>(&h0); r.y = *reinterpret_cast<uint32_t*>(&h1);
                  r.z = *reinterpret_cast<uint32_t*>(&h2); r.w = *reinterpret_cast<uint32_t*>(&h3);
                  dst[c] = r;
                }
              }
            } else if (xr < p.M) {
#pragma unroll
              for (int c = 0; c < CH; ++c) {
                const int n = y0 + c0 + c;
                if (n < p.N) {
                  const size_t o = (size_t)xr * p.ldo + n;
                  float r = v[c] + (p.bias ? p.bias[n] : 0.f);
                  if (p.out_f32) {
                    float* dst = (float*)p.out + o;
                    if (p.epilogue == kAccumulate) r += *dst;
                    *dst = r;
                  } else {
                    ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(r);
                  }
                }
              }
            }
          }
        }
        if (whole) {
          tcgen05_fence_before();
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tempty0 + 8 * b) : "memory");
        }
      }
    }
    if (!SWAP && p.cluster > 1) {
      if (!met_cluster) cluster_sync_all();            // a thread that gave up still meets its peers
      cluster_sync_all();                              // nobody leaves while a peer may still read its share
    }
    if (!SWAP && p.tma_out) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the staging block is read, the stores are done
  }
  if (SWAP && p.cluster > 1 && !push) {
    // The S CTAs of a cluster hold the S consecutive K ranges of one tile.  CTA r adds, in the
    // order of increasing K, the shares of its 1/S of the tile's rows and writes them out.
    cluster_sync_all();
    if (warp >= 2 && flags[0] == 0) {
      const int S = p.cluster;
      const int r = (int)cluster_rank();
      const long long tile = blockIdx.x / S;
      const int x0 = (int)(tile % p.tiles_x) * kTileX, y0 = (int)(tile / p.tiles_x) * BN;
      const bool sw = p.epilogue == kSwiGLU;
      const int rows_per = (sw ? 64 : kTileX) / S;          // rows (gate rows) of this CTA
      const int t = threadIdx.x - 64;
      const int row = r * rows_per + t % rows_per;
      const int cstep = 128 / rows_per;
      const int n = sw ? (x0 / kTileX) * 64 + row : x0 + row;   // output feature
      const int n_end = sw ? p.N / 2 : p.N;
      const float bv = (p.bias && n < n_end) ? p.bias[n] : 0.f;
      constexpr int kCols = 4;                                  // columns a thread has in flight
      for (int cb = t / rows_per; cb < BN; cb += cstep * kCols) {
        float acc[kCols], up[kCols], old[kCols];
#pragma unroll
        for (int j = 0; j < kCols; ++j) {
          const int m = y0 + cb + j * cstep;
          acc[j] = 0.f; up[j] = 0.f;
          old[j] = (p.epilogue == kAccumulate && cb + j * cstep < BN && m < p.M && n < n_end)
                       ? __ldcg((const float*)p.out + (size_t)m * p.ldo + n) : 0.f;
        }
        // every peer's share is requested before the first is used; the sums run in K order
        for (int part = 0; part < (sw ? 2 : 1); ++part) {
          float share[8][kCols];
#pragma unroll
          for (int q = 0; q < 8; ++q)
#pragma unroll
            for (int j = 0; j < kCols; ++j) {
              const int c = cb + j * cstep;
              share[q][j] = (q < S && c < BN)
                                ? ld_peer_f32(base + (uint32_t)(c * kTileX + part * 64 + row) * 4u, (uint32_t)q) : 0.f;
            }
#pragma unroll
          for (int q = 0; q < 8; ++q)
#pragma unroll
            for (int j = 0; j < kCols; ++j) {
              if (part == 0) acc[j] += share[q][j]; else up[j] += share[q][j];
            }
        }
#pragma unroll
        for (int j = 0; j < kCols; ++j) {
          const int c = cb + j * cstep, m = y0 + c;
          if (c < BN && m < p.M && n < n_end) {
            const float g = acc[j];
            const float v = sw ? silu_mul(g, up[j]) : g + bv + old[j];
            const size_t o = (size_t)m * p.ldo + n;
            if (p.out_f32) ((float*)p.out)[o] = v; else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
          }
        }
      }
    }
    cluster_sync_all();                  // nobody leaves while a peer may still read its shares
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ many tokens: pairs of CTAs
// A tile of 256 tokens x 256 weight rows belongs to a cluster of two CTAs on the two SMs of a
// TPC, which the tensor cores treat as one unit (tcgen05.mma.cta_group::2, M = 256): each CTA
// loads its own 128 token rows and its own HALF of the weight block, so a weight byte crosses
// from L2 into one of the two SMs only, a stage is 32 KB instead of 64 (six stages), and each
// CTA's 128 x 256 accumulator takes half of its tensor memory, so the write-out of a tile runs
// under the MMAs of the next one.  One thread of the leader (rank 0) issues for both SMs.
//   full[s]   (leader)  one arrival with 64 KB expected: the loads of BOTH CTAs count here
//   empty[s]  (each)    the leader's commit, sent to both CTAs
//   tfull[b]  (each)    the leader's commit after a tile's last MMA, sent to both CTAs
//   tempty[b] (leader)  two arrivals, one per CTA, when its epilogue has read accumulator b
// Items are (tile, K range): first the tiles of the whole rounds, one item each, then the tiles
// left over, each cut into `split` equal K ranges (all ranges 0, then all ranges 1, ...).  Only
// products that add into a 32-bit output are cut; their ranges meet in memory through the TMA
// reduce of the write-out.
constexpr int kPairStages = 6;
constexpr int kPairN = 256;
constexpr uint32_t kPairBytesA = kTileX * kBlockK * 2, kPairBytesB = (kPairN / 2) * kBlockK * 2;
constexpr uint32_t kPairStageBytes = kPairBytesA + kPairBytesB;
constexpr uint32_t kPairStaging = 2 * kTileX * 128;      // two blocks: one is read by TMA while the next is filled
constexpr size_t kPairSmem = (size_t)kPairStages * kPairStageBytes + kPairStaging + 1024 + (2 * kPairStages + 8) * 8;

struct PairParams {
  const float* bias;
  int* error_flag;
  int M, N;
  int tiles_m;               // 256-token tiles; tile = column tile * tiles_m + token tile
  int k_blocks;              // K blocks of the product
  int n_whole, rest, split;  // tiles that are one item each; tiles cut into `split` K ranges
  int n_items;               // n_whole + rest * split
  int epilogue, out_f32;
};

__global__ void __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                 const __grid_constant__ CUtensorMap map_out, const PairParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes + kPairStaging);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kPairStages;
  const uint32_t tfull0 = empty0 + 8 * kPairStages, tempty0 = tfull0 + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kPairStages + 4);
  volatile int* flags = reinterpret_cast<volatile int*>(bars + 2 * kPairStages + 5);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 2); }
    flags[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  cluster_sync_all();                    // both CTAs' barriers are ready before anything is sent to them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // item -> first token row of the pair's tile, first weight row, K range
  auto place = [&](int item, int& x0, int& y0, int& kb0, int& cnt) {
    int tile = item, ks = 0, s = 1;
    if (item >= p.n_whole) {
      const int j = item - p.n_whole;
      tile = p.n_whole + j % p.rest; ks = j / p.rest; s = p.split;
    }
    x0 = (tile % p.tiles_m) * 2 * kTileX; y0 = (tile / p.tiles_m) * kPairN;
    kb0 = (int)((long long)ks * p.k_blocks / s);
    cnt = (int)((long long)(ks + 1) * p.k_blocks / s) - kb0;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      const uint32_t lead_full0 = peer_addr(full0, 0);
      bool ok = true;
      uint32_t it = 0;
      // The weight depends on no earlier kernel: the weight halves of the first ring are
      // requested before this kernel waits for its predecessor, the token rows after.
      uint32_t early = 0;
      for (int item = pair; item < p.n_items && early < (uint32_t)kPairStages; item += n_pairs) {
        int x0, y0, kb0, cnt;
        place(item, x0, y0, kb0, cnt);
        for (int i = 0; i < cnt && early < (uint32_t)kPairStages; ++i, ++early) {
          if (leader) mbar_expect_tx(full0 + 8 * early, 2 * kPairStageBytes);
          tma_load_2d_pair(base + early * kPairStageBytes + kPairBytesA, &map_y, lead_full0 + 8 * early, (kb0 + i) * kBlockK,
                           y0 + (int)rank * (kPairN / 2));
        }
      }
      pdl_wait();
      for (int item = pair; ok && item < p.n_items; item += n_pairs) {
        int x0, y0, kb0, cnt;
        place(item, x0, y0, kb0, cnt);
        for (int i = 0; i < cnt; ++i, ++it) {
          const uint32_t s = it % kPairStages;
          const uint32_t dst = base + s * kPairStageBytes;
          const int kcol = (kb0 + i) * kBlockK;
          if (it >= early) {
            ok = mbar_wait(empty0 + 8 * s, ((it / kPairStages) - 1) & 1);
            if (!ok) break;
            if (leader) mbar_expect_tx(full0 + 8 * s, 2 * kPairStageBytes);
            tma_load_2d_pair(dst + kPairBytesA, &map_y, lead_full0 + 8 * s, kcol, y0 + (int)rank * (kPairN / 2));
          }
          tma_load_2d_pair(dst, &map_x, lead_full0 + 8 * s, kcol, x0 + (int)rank * kTileX);
        }
      }
      if (!ok) { flags[0] = 1; if (p.error_flag) *p.error_flag = 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (the leader's)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = instr_desc(2 * kTileX, kPairN);
      bool ok = true;
      uint32_t it = 0, n = 0;
      for (int item = pair; ok && item < p.n_items; item += n_pairs, ++n) {
        int x0, y0, kb0, cnt;
        place(item, x0, y0, kb0, cnt);
        const uint32_t b = n & 1;
        ok = mbar_wait(tempty0 + 8 * b, ((n >> 1) & 1) ^ 1);      // both epilogues have read this accumulator
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t acc = tmem_base + b * kPairN;
        for (int i = 0; i < cnt; ++i, ++it) {
          const uint32_t s = it % kPairStages;
          ok = mbar_wait(full0 + 8 * s, (it / kPairStages) & 1);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a = base + s * kPairStageBytes;
          const uint64_t da = smem_desc(a), db = smem_desc(a + kPairBytesA);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k)
            mma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit_pair(empty0 + 8 * s, (uint16_t)3);
        }
        if (ok) tcgen05_commit_pair(tfull0 + 8 * b, (uint16_t)3);
      }
      if (!ok) {
        flags[0] = 1; if (p.error_flag) *p.error_flag = 1;
        tcgen05_commit_pair(tfull0, (uint16_t)3); tcgen05_commit_pair(tfull0 + 8, (uint16_t)3);   // let the epilogues leave their waits
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t stg0 = base + kPairStages * kPairStageBytes;
    const uint32_t lead_tempty0 = peer_addr(tempty0, 0);
    const bool elected = row == 0;
    uint32_t n = 0, flushes = 0;
    pdl_wait();                               // the output belongs to earlier kernels until now
    for (int item = pair; item < p.n_items; item += n_pairs, ++n) {
      int x0, y0, kb0, cnt;
      place(item, x0, y0, kb0, cnt);
      const uint32_t b = n & 1;
      if (!mbar_wait(tfull0 + 8 * b, (n >> 1) & 1)) { flags[0] = 1; if (p.error_flag) *p.error_flag = 1; }
      tcgen05_fence_after();
      if (flags[0] != 0) break;
      const int xr0 = x0 + (int)rank * kTileX;              // first output row of this CTA's half
      const bool rows_live = xr0 < p.M;
      const bool with_bias = p.bias != nullptr && kb0 == 0;  // of the ranges that meet in memory, the first adds it
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + b * kPairN;
      auto flush_row = [&](const uint4 (&piece)[8], int out_col) {
        const uint32_t stg = stg0 + (flushes++ & 1u) * (kTileX * 128u);
        if (elected) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");     // this block's last reader is done (the other's may still run)
        asm volatile("bar.sync 2, 128;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg + (uint32_t)row * 128u + (uint32_t)((j ^ (row & 7)) << 4)),
                       "r"(piece[j].x), "r"(piece[j].y), "r"(piece[j].z), "r"(piece[j].w) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (elected) {
          // (a half that lies wholly beyond M still commits a group, empty, so that the count above holds)
          if (!rows_live) {}
          else if (p.epilogue == kAccumulate)
            asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&map_out), "r"(stg), "r"(out_col), "r"(xr0) : "memory");
          else
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&map_out), "r"(stg), "r"(out_col), "r"(xr0) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      };
      auto pack8 = [&](const float* r8) {
        uint4 q;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(r8[0], r8[1]), h1 = __floats2bfloat162_rn(r8[2], r8[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(r8[4], r8[5]), h3 = __floats2bfloat162_rn(r8[6], r8[7]);
        q.x = *reinterpret_cast<uint32_t*>(&h0); q.y = *reinterpret_cast<uint32_t*>(&h1);
        q.z = *reinterpret_cast<uint32_t*>(&h2); q.w = *reinterpret_cast<uint32_t*>(&h3);
        return q;
      };
      uint4 piece[8];
      if (p.epilogue == kSwiGLU) {
        // columns come in blocks of 64 gate then 64 up: 64 outputs = one 128-byte row of bf16
        for (int cb = 0; cb < kPairN; cb += 128) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            float g[32], u[32], r[32];
            tmem_load_32(taddr + cb + 32 * half, g);
            tmem_load_32(taddr + cb + 64 + 32 * half, u);
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = silu_mul(g[c], u[c]);
#pragma unroll
            for (int j = 0; j < 4; ++j) piece[4 * half + j] = pack8(r + 8 * j);
          }
          flush_row(piece, (y0 + cb) / 2);
        }
      } else if (p.out_f32) {
        for (int c0 = 0; c0 < kPairN; c0 += 32) {
          float v[32];
          tmem_load_32(taddr + c0, v);
          if (with_bias) {
#pragma unroll
            for (int c = 0; c < 32; ++c) v[c] += (y0 + c0 + c < p.N) ? p.bias[y0 + c0 + c] : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            piece[j] = make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
          flush_row(piece, y0 + c0);
        }
      } else {
        for (int c0 = 0; c0 < kPairN; c0 += 64) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            float v[32];
            tmem_load_32(taddr + c0 + 32 * half, v);
            if (p.bias) {
#pragma unroll
              for (int c = 0; c < 32; ++c) v[c] += (y0 + c0 + 32 * half + c < p.N) ? p.bias[y0 + c0 + 32 * half + c] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) piece[4 * half + j] = pack8(v + 8 * j);
          }
          flush_row(piece, y0 + c0);
        }
      }
      // the accumulator is read: one arrival per CTA tells the leader's issuer
      tcgen05_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        if (leader) mbar_arrive(tempty0 + 8 * b); else mbar_arrive_cluster(lead_tempty0 + 8 * b);
      }
    }
    if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the staging block is read, the stores are done
  }
  __syncwarp();
  tcgen05_fence_before();
  cluster_sync_all();                    // nobody leaves while its peer may still signal it or use its memory
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* ptr; int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    for (int v : {k.rows, k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ std::hash<int>()(v);
    return h;
  }
};

// A [rows, cols] bf16 matrix with leading dimension ld (elements); box = [box_rows, 64].
int make_map(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail("gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows %d cols %d ld %d)", (int)r, rows, cols, ld);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// The [rows, cols] output (32-bit or bf16, leading dimension ld elements); box = 128 rows x 128 bytes.
int make_out_map(CUtensorMap* out, const void* ptr, int rows, int cols, int ld, bool f32) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  const MapKey key{ptr, rows, cols, ld, f32 ? 4 : 2};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail("gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
  const int es = f32 ? 4 : 2;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * es};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / es), (cuuint32_t)kTileX};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("gemm_tc: cuTensorMapEncodeTiled failed with code %d for the output (rows %d cols %d ld %d)", (int)r, rows, cols, ld);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

// Ring, alignment slack, barriers and flags, then the exchange area: the whole-tile SwiGLU
// exchange, or (`sent`) the shares that the CTAs of a cluster send here.
template <int BN, int STAGES, bool SWAP, int MS = 1>
constexpr size_t smem_bytes(bool sent = true) {
  return (size_t)STAGES * (MS * kTileX * kBlockK * 2 + BN * kBlockK * 2) + 1024 + (2 * STAGES + 8) * 8 +
         (SWAP ? 0 : MS * kTileX * 128) +       // many tokens: the staging block of each row block
         (SWAP ? (sent && BN <= 64 && kTileX * BN * 4 > 32 * 64 * 4 ? kTileX * BN * 4 : 32 * 64 * 4) : 0);
}

template <int BN, int STAGES, bool SWAP, int MS = 1>
int configure() {
  constexpr size_t smem = smem_bytes<BN, STAGES, SWAP, MS>();
  static_assert(smem <= 227 * 1024, "stage ring does not fit shared memory");
  static OncePerDevice once;
  if (once.first()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SWAP, MS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) once.forget();
    if (e != cudaSuccess) return fail("gemm_tc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    // two CTAs of the small rings share an SM only with the largest shared-memory carve-out
    cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, SWAP, MS>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  return 0;
}

// How many clusters of `split` CTAs of this kernel the device holds at a time (0 if unknown).
template <int BN, int STAGES, bool SWAP>
int active_clusters(int split) {
  static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (split < 1 || split > 8) return 0;
  if (cache[split] != 0) return cache[split] < 0 ? 0 : cache[split];
  if (configure<BN, STAGES, SWAP>()) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(split * 256);
  cfg.blockDim = dim3(threads_for(1));
  cfg.dynamicSmemBytes = smem_bytes<BN, STAGES, SWAP>();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BN, STAGES, SWAP, 1>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cache[split] = n > 0 ? n : -1;
  return n > 0 ? n : 0;
}

int active_clusters_for(int bn, int split) {
  switch (bn) {
    case 16: return active_clusters<16, 5, true>(split);
    case 32: return active_clusters<32, 4, true>(split);
    case 64: return active_clusters<64, 3, true>(split);
    default: return active_clusters<128, 3, true>(split);
  }
}

template <int BN, int STAGES, bool SWAP, int MS = 1>
int launch(const CUtensorMap& mx, const CUtensorMap& my, const CUtensorMap& mo, const Params& p, int grid, cudaStream_t stream) {
  const size_t smem = smem_bytes<BN, STAGES, SWAP, MS>(p.cluster > 1);
  if (configure<BN, STAGES, SWAP, MS>()) return -1;
  ilb::launch_cluster(gemm_tc_kernel<BN, STAGES, SWAP, MS>, dim3(grid), dim3(threads_for(MS)), smem, stream, p.cluster, mx, my, mo, p);
  return check_launch("gemm_tc");
}

}  // namespace

// Elements of 32-bit workspace and tickets a call may need, for the caller to allocate:
// two slots of a whole tile (up to 256 x 256) per CTA of the largest persistent grid (one
// CTA per SM for those tiles), one ticket per output tile.
ILB_EXPORT long long ilb_gemm_tc_workspace_floats() {
  const long long ctas = sm_count() > 152 ? sm_count() : 152;
  return 2ll * ctas * 256 * 256;
}
ILB_EXPORT int ilb_gemm_tc_max_tickets() { return 1 << 16; }

// Clusters of `split` CTAs of the decode kernel for token tiles of `bn` that fit the device at once.
ILB_EXPORT int ilb_gemm_tc_active_clusters(int bn, int split) { return active_clusters_for(bn, split); }
// What the kernel can take: bf16 operands, K and the leading dimensions multiples of 8
// (16-byte rows for TMA), 16-byte aligned bases.
ILB_EXPORT int ilb_gemm_tc_supported(int M, int N, int K, int lda, int ldw) {
  return (M > 0 && N > 0 && K > 0 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0) ? 1 : 0;
}

namespace {
// How a product is dealt out: orientation, tile shape, grid, cluster, rounds (fills the
// scheduling fields of `p`, which must hold M, N, K, k_blocks and the epilogue already).
struct Plan { bool swap, tail, additive; int bn, ms, x_rows, y_rows; long long grid; };

// Whether the K ranges of a tile may meet in memory (the sum's order is then not fixed: runs
// agree beyond rounding, not bit for bit).  `ilb_gemm_tc_sums_in_memory(0)` turns it off.
bool g_sums_in_memory = true;
// Accumulating products of up to this many tokens, with a weight of at least 2,048 x 2,048, add
// the K ranges of a tile in memory (separate CTAs, red.add) instead of inside a cluster.  In a
// decode step of Qwen3-8B sizes, one 32-bit value per add: batch 1 3.41 -> 3.31 ms, batch 2
// 3.44 -> 3.36, batch 4 3.51 -> 3.47, but batch 8 3.62 -> 3.70 and batch 16 3.92 -> 4.26 (the
// adds are paid per lane); four neighbouring features per add (the share transposed through
// shared memory): batch 1 3.29, batch 4 3.43, batch 8 3.52 ms.
int g_red_few_tokens = 8;
int g_red_few_split = 8;

// Equal K ranges per tile when `rest` tiles share the SMs: as many as fit, none shorter than
// four K blocks.
long long add_split(long long rest, long long k_blocks) {
  long long split = sm_count() / rest;
  if (split > k_blocks / 4) split = k_blocks / 4;
  return split < 1 ? 1 : split;
}

// `can_add`: the product accumulates into a 32-bit output that the TMA write-out can reach,
// so that the K ranges of a tile may be added in memory.
int make_plan(Params& p, int M, int N, int K, int accumulate, int n_tickets, int max_ctas, bool can_add, Plan& plan) {
  // 65 to 128 tokens of a product that accumulates into a wide 32-bit output: tokens on the
  // MMA's rows after all, 128 x 256 tiles cut into equal K ranges that meet in memory.  With
  // the weight on the rows the K ranges of a tile are a cluster that exchanges 32-bit shares;
  // here nothing is exchanged (4,096 x 4,096 at 128 tokens 16.4 -> 12.7 us, 5,120 x 25,600 at
  // 64 tokens 56.0 -> 46.3 us alone; but inside a decode step, between its neighbours, the
  // weight on the rows stays ahead up to 64 tokens: 5.86 against 5.90 ms at batch 64, and
  // 8.35 against 7.86 ms at batch 96).
  bool few_in_memory = false;
  if (M > 64 && M <= 128 && can_add && accumulate == 1 && g_sums_in_memory && max_ctas <= 0 && N >= 3072) {
    const long long t = (N + 255) / 256, kb = (K + kBlockK - 1) / kBlockK;
    const long long rest = t % sm_count();
    few_in_memory = rest != 0 && t * 12 >= sm_count() && add_split(rest, kb) >= 2;
  }
  const bool swap = M <= 128 && !few_in_memory;
  bool tail = false;
  int bn, ms = 1;                                    // ms: 128-row blocks of X per tile
  if (few_in_memory) {
    bn = 256;
    tail = true;
  } else if (swap) {
    bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  } else {
    // Many tokens: the tile shape that keeps the most SMs busy in whole rounds, larger tiles
    // counting for more because they move fewer bytes per flop.
    // Few tiles are cut into equal K ranges; with one 128-row block per tile the ranges of a
    // tile run as a cluster that shares the write-out, with two they go through a ticket.
    // (160 columns: 32 column tiles for a width of 5120, where 256 and 192 leave a quarter of
    // the SMs idle; its 32-bit write-out goes in 32-column pieces, the 16-bit one needs 64)
    const struct { int ms, bn; double worth; } shapes[7] = {{2, 256, 1.0}, {2, 192, 0.93}, {2, 160, 0.9}, {1, 256, 0.85},
                                                            {1, 192, 0.8}, {1, 160, 0.78}, {1, 128, 0.7}};
    const long long kb = (K + kBlockK - 1) / kBlockK;
    double best = -1.0;
    bn = 128;
    for (const auto& c : shapes) {
      if (c.bn > 128 && N < 256) continue;
      if (c.bn % 128 != 0 && accumulate == 2) continue;        // the SwiGLU epilogue pairs 64-column blocks
      if (c.bn % 64 != 0 && !(p.out_f32 || accumulate == 1)) continue;   // 16-bit results leave in 64-column pieces
      const long long tm = (M + c.ms * kTileX - 1) / (c.ms * kTileX), tn = (N + c.bn - 1) / c.bn;
      const long long t = tm * tn;
      // the part of the tiles' area that holds real rows and columns
      const double filled = ((double)M / (double)(tm * c.ms * kTileX)) * ((double)N / (double)(tn * c.bn));
      double score;
      if ((c.bn == 160 || (c.bn == 192 && c.ms == 1)) && t * 2 <= sm_count()) continue;   // (few tiles are cut into K ranges whose CTAs share 32-column pieces of 128 or 256)
      if (t * 2 <= sm_count()) {
        long long split = 1;
        while (split < 8 && t * split * 2 <= sm_count() && split * 2 <= kb) split *= 2;
        score = (double)(t * split) / sm_count() * c.worth * (c.ms == 1 ? 0.9 : 0.6);
      } else {
        const long long rounds = (t + sm_count() - 1) / sm_count();
        score = (double)t / (double)(rounds * sm_count()) * c.worth;
      }
      score *= filled;
      if (score > best) { best = score; bn = c.bn; ms = c.ms; }
    }
    // A short last round: the tiles left over after the whole rounds (all of them, when they
    // are fewer than the SMs) are each cut into as many equal K ranges as the SMs allow, so the
    // last round is as short as its tiles are few and the largest tile serves whatever the
    // sizes.  (Equal ranges, not equal runs over all the tiles' K blocks: CTAs that share an
    // operand block must reach it together, or each streams its own copy from memory.)  Only
    // where the product accumulates into a 32-bit output: there the ranges of a tile meet in
    // memory at the cost of a second write-out.  (Through the workspace and a ticket instead,
    // for the other epilogues, the last round's 32-bit round trip cost more than the idle SMs:
    // 30 -> 47 us for 512 x 6144 x 4096, 113 -> 166 us for 2048 x 7168 x 5120.)
    // (Not for a handful of tiles: there it gains little, and small products keep sums whose
    // bits do not change from run to run.)
    if (can_add && g_sums_in_memory && accumulate == 1 && max_ctas <= 0 && N >= 256) {
      for (int cms = 2; cms >= 1; --cms) {
        const long long tm = (M + cms * kTileX - 1) / (cms * kTileX), tn = (N + 255) / 256, t = tm * tn;
        const long long rounds = t / sm_count(), rest = t - rounds * sm_count();
        if (rest == 0 || t * 12 < sm_count()) continue;            // whole rounds, or a product of a handful of tiles
        const long long split = add_split(rest, kb);
        if (split < 2) continue;
        const double filled = ((double)M / (double)(tm * cms * kTileX)) * ((double)N / (double)(tn * 256));
        const double time = (double)rounds + 1.0 / (double)split + 0.03;      // in tile times; the last term: a second write-out
        const double score = (cms == 2 ? 1.0 : 0.95) * filled * ((double)t / (double)sm_count()) / time;
        if (score > best) { best = score; bn = 256; ms = cms; tail = true; }
      }
    }
  }
  const int x_rows = swap ? N : M, y_rows = swap ? M : N;
  p.tiles_x = (x_rows + ms * kTileX - 1) / (ms * kTileX);
  p.tiles_y = (y_rows + bn - 1) / bn;
  const long long tiles = (long long)p.tiles_x * p.tiles_y;
  ILB_REQUIRE(tiles <= n_tickets, "gemm_tc: %lld output tiles exceed the %d tickets", tiles, n_tickets);

  // Decode shapes (swap): two CTAs per SM (the rings are sized for it), one streams while
  // the other is in its prologue or epilogue.  When the tiles are fewer than the CTAs that
  // fit, every tile is cut into the same number of K ranges (at most 8), so that no CTA
  // straddles two tiles; otherwise the persistent grid takes contiguous runs of units.
  const long long cap = swap ? 2ll * sm_count() : sm_count();
  long long grid = cap;
  p.cluster = 1;
  if (swap && tiles <= cap && max_ctas <= 0) {
    // every tile is cut into 1, 2, 4 or 8 K ranges, one per CTA of a cluster that adds them
    // through shared memory: no workspace round trip and no tickets
    long long split = 1;
    while (split < 8 && tiles * split * 2 <= cap && split * 2 <= p.k_blocks) split *= 2;
    // All clusters resident at once, or the stragglers cost a second round.  The occupancy
    // query counts one CTA of this kernel per SM; the small rings run two per SM, and then a
    // cluster of `split` CTAs takes the SMs of a cluster of split / 2.
    const bool two_per_sm = true;
    while (split > 1 && active_clusters_for(bn, (int)(two_per_sm ? split / 2 : split)) < tiles) split /= 2;
    grid = tiles * split;
    p.cluster = (int)split;
    if (can_add && g_sums_in_memory && accumulate == 1 && M <= g_red_few_tokens && split > 1 && N >= 2048 && K >= 2048) {
      // the ranges as separate CTAs that add into the output (as many as the cluster would have held, or more)
      long long s = split;
      while (s < g_red_few_split && tiles * s * 2 <= cap && s * 2 <= p.k_blocks) s *= 2;
      grid = tiles * s;
      p.cluster = 1;
      p.red_out = 1;
    }
  }
  if (!swap && max_ctas <= 0) {
    // Many tokens.  Tiles that share an operand block must want it at the same time, or every
    // CTA streams its own copy from memory: whole tiles in rounds of equal size, all CTAs
    // of a round starting at K block 0 together; when the tiles would leave most SMs idle,
    // every tile is cut into the same number of K ranges instead.
    const long long sms = sm_count();
    if (tail) {
      p.dp_waves = (int)(tiles / sms);
      p.sk_tile0 = (long long)p.dp_waves * sms;
      const long long rest = tiles - p.sk_tile0;
      p.sk_ctas = (int)(rest * add_split(rest, p.k_blocks));
      grid = p.dp_waves > 0 ? sms : p.sk_ctas;
    } else if (tiles * 2 <= sms) {
      long long split = 1;
      while (split < 8 && tiles * split * 2 <= sms && split * 2 <= p.k_blocks) split *= 2;
      if (ms == 1 && split > 1) {
        // the K ranges of a tile as one cluster (all resident, or a second round costs more than it saves)
        while (split > 1 && (bn == 256 ? active_clusters<256, 4, false>((int)split) : active_clusters<128, 6, false>((int)split)) < tiles)
          split /= 2;
        while (split > 1 && bn / split < 32) split /= 2;        // a CTA writes out whole 32-column chunks
        if (accumulate == 2) while (split > 1 && (bn / split) % 128 != 0) split /= 2;   // SwiGLU pairs 64-column blocks
        p.cluster = (int)split;
      }
      grid = tiles * split;
      p.dp_waves = 0;
      p.sk_tile0 = 0;
    } else {
      const long long rounds = (tiles + sms - 1) / sms;
      grid = (tiles + rounds - 1) / rounds;
      p.dp_waves = (int)rounds;
      p.sk_tile0 = tiles;
    }
  } else {
    if (max_ctas > 0) grid = max_ctas;       // tests and tuning runs choose the grid themselves
    if (grid > tiles * p.k_blocks) grid = tiles * p.k_blocks;
    // whole tiles in wave order first, the last partial wave stream-K; decode shapes: everything stream-K
    p.dp_waves = swap ? 0 : (int)(tiles / grid);
    p.sk_tile0 = (long long)p.dp_waves * grid;
  }
  p.units = (tiles - p.sk_tile0) * p.k_blocks;
  plan.swap = swap; plan.tail = tail; plan.additive = tail && can_add && accumulate == 1; plan.bn = bn; plan.ms = ms; plan.x_rows = x_rows; plan.y_rows = y_rows; plan.grid = grid;
  return 0;
}

// ---- pairs of CTAs: how many pairs the device holds at once, the K ranges per tile, the launch
int pair_capacity() {
  static int cached = 0;
  if (cached != 0) return cached < 0 ? 0 : cached;
  if (cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairSmem) != cudaSuccess) {
    cudaGetLastError(); cached = -1; return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 256);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = kPairSmem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cached = n > 0 ? n : -1;
  return n > 0 ? n : 0;
}

// 0: never; 1: where the sizes favour it (the default); 2: wherever the kernel can run (tests).
int g_pairs = 1;
int g_pair_split_max = 8;       // tuning runs lower it

struct PairPlan { int n_whole, rest, split, n_pairs; long long items; double fill; bool few; };

// How the tiles of a product are dealt to the pairs.  Every tile one item, in rounds of equal
// size; or (where the ranges may meet in memory) every tile cut into the same number of K
// ranges; or whole rounds on every pair and the tiles left over cut so that their ranges
// fill one more, shorter, round.  The modelled time, in tile times: rounds of whole tiles,
// plus rounds of ranges / ranges per tile, plus what the extra write-outs cost: every range
// adds a whole 256 x 256 tile of 32-bit values into memory, and those additions share one
// throughput (measured: three ranges per tile of a 4,096 x 5,120 x 5,120 product cost 22 %
// more than their MMA time says; the charge below is half of 0.13 us per extra tile over the
// tile's own 0.4 us per K block).  No range shorter than 16 K blocks.
// `fill`: the time of a perfect deal over the modelled one.
bool pair_plan(int M, int N, int K, bool can_split, int capacity, PairPlan& out) {
  if (capacity <= 0) return false;
  const long long t = (long long)((M + 2 * kTileX - 1) / (2 * kTileX)) * ((N + kPairN - 1) / kPairN);
  const int kb = (K + kBlockK - 1) / kBlockK;
  const int s_max = can_split ? (kb / 16 < g_pair_split_max ? (kb / 16 < 1 ? 1 : kb / 16) : g_pair_split_max) : 1;
  double best = 1e30;
  auto take = [&](double time, long long n_whole, long long rest, int s, long long pairs) {
    time += 0.5 * (double)(rest * (s - 1)) * 0.13 / (0.4 * kb);
    if (time < best - 1e-9) {
      best = time;
      out.n_whole = (int)n_whole; out.rest = (int)rest; out.split = s; out.n_pairs = (int)pairs; out.items = n_whole + rest * s;
    }
  };
  for (int s = 1; s <= s_max; ++s) {                       // every tile cut alike
    const long long items = t * s, rounds = (items + capacity - 1) / capacity;
    take((double)rounds / s, 0, t, s, (items + rounds - 1) / rounds);
  }
  const long long whole = t / capacity, rest = t % capacity;
  if (whole > 0 && rest > 0) {                             // whole rounds, then one round of ranges
    int s = (int)(capacity / rest);
    if (s > s_max) s = s_max;
    if (s > 1) take((double)whole + 1.0 / s, whole * capacity, rest, s, capacity);
  }
  // (tiles of 256 tokens hold more empty rows than blocks of 128 would when M leaves the odd block empty)
  const double rows = (double)((M + kTileX - 1) / kTileX * kTileX) / (double)((M + 2 * kTileX - 1) / (2 * kTileX) * (2 * kTileX));
  out.fill = ((double)t / capacity) / best * rows;
  out.few = t < capacity;
  return true;
}

// Pairs where the deal keeps them busy: products that add into the 32-bit output have the
// single-CTA tiles' short last round as the alternative, so they ask for more, except where
// the tiles are fewer than the pairs (there the single-CTA tiles have no whole round either).
double g_pair_fill_plain = 0.75, g_pair_fill_adding = 0.85;
bool pair_wanted(const PairPlan& pp, int epilogue) {
  if (g_pairs == 2) return true;
  if (epilogue == 1) return pp.fill >= g_pair_fill_adding || (pp.few && pp.split > 1);
  return pp.fill >= g_pair_fill_plain;
}

int launch_pair(const CUtensorMap& mx, const CUtensorMap& my, const CUtensorMap& mo, const PairParams& p, int n_pairs, cudaStream_t stream) {
  static OncePerDevice once;
  if (once.first()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairSmem);
    if (e != cudaSuccess) { once.forget(); return fail("gemm_tc: cannot reserve %zu bytes of shared memory: %s", kPairSmem, cudaGetErrorString(e)); }
  }
  ilb::launch_cluster(gemm_pair_kernel, dim3(2 * n_pairs), dim3(192), kPairSmem, stream, 2, mx, my, mo, p);
  return check_launch("gemm_tc");
}

}  // namespace

// max_ctas > 0 sets the grid (tests use it to force many shared tiles).
ILB_EXPORT int ilb_gemm_tc(const void* A, const void* W, const float* bias, void* out, int out_f32,
                           int M, int N, int K, int lda, int ldw, int ldo, int accumulate /* Epilogue */,
                           float* workspace, long long workspace_floats, int* tickets, int n_tickets,
                           int* error_flag, int max_ctas, cudaStream_t stream) {
  ILB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  ILB_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
              "gemm_tc: K (%d) and the leading dimensions (%d, %d) must be multiples of 8", K, lda, ldw);
  ILB_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tc: operands must be 16-byte aligned");
  ILB_REQUIRE(accumulate >= 0 && accumulate <= 2, "gemm_tc: unknown epilogue %d", accumulate);
  ILB_REQUIRE(accumulate != 1 || out_f32, "gemm_tc: accumulation needs a 32-bit output");
  if (accumulate == 2) {
    ILB_REQUIRE(N % 128 == 0 && bias == nullptr, "gemm_tc: the SwiGLU epilogue needs N (%d) a multiple of 128 and no bias", N);
    ILB_REQUIRE(ldo >= N / 2, "gemm_tc: output leading dimension too small");
  } else {
    ILB_REQUIRE(ldo >= N, "gemm_tc: output leading dimension too small");
  }
  ILB_REQUIRE(workspace != nullptr && tickets != nullptr, "gemm_tc: workspace and tickets are required");

  Params p{};
  p.out = out; p.bias = bias; p.partial = workspace; p.tickets = tickets; p.error_flag = error_flag;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo;
  p.k_blocks = (K + kBlockK - 1) / kBlockK;
  p.epilogue = accumulate;
  p.out_f32 = out_f32;

  Plan plan{};
  const int es = out_f32 ? 4 : 2, out_cols = accumulate == 2 ? N / 2 : N;
  const bool tma_reach = ((uintptr_t)out % 16 == 0) && ((long long)ldo * es) % 16 == 0;   // rows of 16-byte multiples from a 16-byte base
  if (make_plan(p, M, N, K, accumulate, n_tickets, max_ctas, tma_reach && out_f32 && accumulate == 1, plan)) return -1;
  const bool swap = plan.swap;
  // Many tokens: a pair of CTAs per 256 x 256 tile where the result can leave by TMA.
  if (!swap && g_pairs != 0 && max_ctas <= 0 && tma_reach && !(accumulate == 2 && out_f32)) {
    PairPlan pp{};
    if (pair_plan(M, N, K, out_f32 && accumulate == 1 && g_sums_in_memory, pair_capacity(), pp) && pair_wanted(pp, accumulate)) {
      PairParams q{};
      q.bias = bias; q.error_flag = error_flag; q.M = M; q.N = N;
      q.tiles_m = (M + 2 * kTileX - 1) / (2 * kTileX);
      q.k_blocks = p.k_blocks; q.n_whole = pp.n_whole; q.rest = pp.rest; q.split = pp.split; q.n_items = (int)pp.items;
      q.epilogue = accumulate; q.out_f32 = out_f32;
      CUtensorMap mx, my, mo;
      if (make_map(&mx, A, M, K, lda, kTileX)) return -1;
      if (make_map(&my, W, N, K, ldw, kPairN / 2)) return -1;
      if (make_out_map(&mo, out, M, out_cols, ldo, out_f32 != 0)) return -1;
      return launch_pair(mx, my, mo, q, pp.n_pairs, stream);
    }
  }
  const int bn = plan.bn, ms = plan.ms, x_rows = plan.x_rows, y_rows = plan.y_rows;
  const long long grid = plan.grid;
  ILB_REQUIRE(swap || p.cluster == 1 || (bn / p.cluster) % 32 == 0, "gemm_tc: %d columns do not divide among %d CTAs", bn, p.cluster);
  ILB_REQUIRE(2 * grid * ms * bn * kTileX <= workspace_floats, "gemm_tc: workspace too small");

  CUtensorMap mx, my;
  const void* X = swap ? W : A;
  const void* Y = swap ? A : W;
  const int ldx = swap ? ldw : lda, ldy = swap ? lda : ldw;
  if (make_map(&mx, X, x_rows, K, ldx, kTileX)) return -1;
  if (make_map(&my, Y, y_rows, K, ldy, bn)) return -1;
  // Many tokens, one CTA per tile's write-out: the result leaves by TMA (rows of 16-byte multiples from a 16-byte base)
  CUtensorMap mo = mx;
  // (a cluster's CTAs each write a share of the columns: whole 128-byte rows of it, or per-thread stores)
  const int share_cols = bn / (p.cluster > 0 ? p.cluster : 1);
  const bool whole_rows = p.cluster == 1 || (accumulate == 2 ? share_cols % 128 == 0 : share_cols % (128 / es) == 0);
  p.tma_out = (!swap && whole_rows && !(accumulate == 2 && out_f32) && tma_reach) ? 1 : 0;
  ILB_REQUIRE(!plan.additive || p.tma_out, "gemm_tc: partial sums that meet in memory need the TMA write-out");
  if (p.tma_out && make_out_map(&mo, out, M, out_cols, ldo, out_f32 != 0)) return -1;

  if (swap) {
    switch (bn) {
      case 16: return launch<16, 5, true>(mx, my, mo, p, (int)grid, stream);
      case 32: return launch<32, 4, true>(mx, my, mo, p, (int)grid, stream);
      // the shares sent to a CTA take the room of a stage: a shallower ring for clusters only
      case 64: return p.cluster > 1 ? launch<64, 3, true>(mx, my, mo, p, (int)grid, stream) : launch<64, 4, true>(mx, my, mo, p, (int)grid, stream);
      default: return launch<128, 3, true>(mx, my, mo, p, (int)grid, stream);
    }
  }
  if (bn == 256 && ms == 2) return launch<256, 3, false, 2>(mx, my, mo, p, (int)grid, stream);
  if (bn == 192 && ms == 2) return launch<192, 3, false, 2>(mx, my, mo, p, (int)grid, stream);
  if (bn == 192) return launch<192, 5, false>(mx, my, mo, p, (int)grid, stream);
  if (bn == 160 && ms == 2) return launch<160, 3, false, 2>(mx, my, mo, p, (int)grid, stream);
  if (bn == 160) return launch<160, 5, false>(mx, my, mo, p, (int)grid, stream);
  if (bn == 256) return launch<256, 4, false>(mx, my, mo, p, (int)grid, stream);
  return launch<128, 6, false>(mx, my, mo, p, (int)grid, stream);
}

// Products of many tokens on pairs of CTAs: 0 never, 1 where the sizes favour it, 2 wherever possible.
ILB_EXPORT int ilb_gemm_tc_pairs(int mode) {
  g_pairs = mode < 0 ? 0 : mode > 2 ? 2 : mode;
  return 0;
}

// Tuning runs: few-token accumulating products of up to `max_tokens` tokens add their K ranges in
// memory instead of inside a cluster, cut into up to `max_split` ranges.
ILB_EXPORT int ilb_gemm_tc_red_few(int max_tokens, int max_split) {
  g_red_few_tokens = max_tokens;
  g_red_few_split = max_split < 1 ? 1 : max_split > 16 ? 16 : max_split;
  return 0;
}

// Tuning runs: the most K ranges a tile of a pair is cut into (1 to 8), and how well the deal
// must fill the pairs (in thousandths) for plain and for adding products.
ILB_EXPORT int ilb_gemm_tc_pair_tuning(int split_max, int fill_plain, int fill_adding) {
  g_pair_split_max = split_max < 1 ? 1 : split_max > 8 ? 8 : split_max;
  g_pair_fill_plain = fill_plain / 1000.0;
  g_pair_fill_adding = fill_adding / 1000.0;
  return 0;
}

// 1: the K ranges of a tile may meet in memory (the default); 0: every split sum is added in K order.
ILB_EXPORT int ilb_gemm_tc_sums_in_memory(int on) {
  g_sums_in_memory = on != 0;
  return 0;
}

// What a product of these sizes would get (for tests and notes): out[0..8] = swapped operands,
// token-tile / weight-tile width, 128-row blocks per tile, grid, cluster, whole-tile rounds,
// tiles, tiles handled stream-K fashion, whether the K ranges of a tile are added in memory;
// out[9..10] = pairs of CTAs and K ranges per tile when the product runs on pairs (else 0, 0;
// an output that TMA cannot reach keeps the single-CTA tiles whatever this says).
ILB_EXPORT int ilb_gemm_tc_plan(int M, int N, int K, int epilogue, int* out) {
  ILB_REQUIRE(M > 0 && N > 0 && K > 0 && out != nullptr && epilogue >= 0 && epilogue <= 2, "gemm_tc: bad sizes for a plan");
  Params p{};
  p.M = M; p.N = N; p.K = K; p.k_blocks = (K + kBlockK - 1) / kBlockK; p.epilogue = epilogue;
  Plan plan{};
  if (make_plan(p, M, N, K, epilogue, 1 << 30, 0, epilogue == 1, plan)) return -1;
  out[0] = plan.swap ? 1 : 0; out[1] = plan.bn; out[2] = plan.ms; out[3] = (int)plan.grid; out[4] = p.cluster;
  out[5] = p.dp_waves; out[6] = p.tiles_x * p.tiles_y; out[7] = (int)(p.tiles_x * (long long)p.tiles_y - p.sk_tile0);
  out[8] = (plan.additive || p.red_out) ? 1 : 0;
  out[9] = 0; out[10] = 0;
  PairPlan pp{};
  if (!plan.swap && g_pairs != 0 && pair_plan(M, N, K, epilogue == 1 && g_sums_in_memory, pair_capacity(), pp) &&
      pair_wanted(pp, epilogue)) {
    out[9] = pp.n_pairs; out[10] = pp.split;
    out[8] = pp.split > 1 ? 1 : 0;
  }
  return 0;
}

ILB_DEFINE_LAST_ERROR()
