// Causal grouped-query prefill attention over the paged bfloat16 cache on the tcgen05
// tensor cores: S = Q K^T and O += P V as tcgen05.mma with both accumulators in tensor
// memory, operands brought by TMA straight from the cache pages.
//
// One CTA = one kv head and 128 rows, a row being a (token, query head of the group)
// pair, so floor(128 / G) tokens of one sequence (a group size that does not divide 128
// leaves the last 128 mod G rows unused: 3 of 128 for groups of 5); it walks that
// sequence's keys 128 at a time.
//   warp 0   looks up the pages of the next 128 keys in the block table and issues the TMA
//            loads: K and V each as one box per page (the tensor map has the key's place in
//            its group of 8, the 64-wide slice of the head and the group as dimensions, so a
//            whole page lands in the operand layout; 128-byte swizzle; a page that is not held
//            is requested outside the tensor, which TMA fills with zeros), or one box for the
//            tile when its pages follow one another in the pool; Q once.
//   warp 1   allocates tensor memory (two S tiles of 128 columns and O of head-size columns);
//            one lane issues S = Q K^T two tiles ahead (tile j+2 goes to the S tile that held
//            tile j, right behind O += P V of tile j: the tensor core runs its operations in the
//            order they were issued), so the tensor core works on tile j+1 and j+2 while the
//            softmax warps are on tile j+1.  P is the MMA's A operand straight from tensor
//            memory; V is used as it lies in the cache ([key][d], the "MN-major" operand
//            form), no transpose.
//   warps 2-9  two threads per row (row = tensor-memory lane, each thread half of the tile's
//            keys): read S into registers, exchange the row maximum through shared memory,
//            keep the running maximum and sum in 32-bit, write P as packed bfloat16 back into
//            the tensor-memory columns S came from (tcgen05.st), and rescale O in tensor
//            memory only when the maximum has grown by more than 2^8 (any fixed reference
//            maximum gives the same quotient; the threshold only bounds the magnitudes).  At
//            the end it divides O by the sum and writes the row.
// Every mbarrier wait is bounded; on expiry a flag is raised, the CTA drains and frees its
// tensor memory.  No cluster, no multicast.
//
// Reference counterparts: the query-tile prefill kernel on MMAs
// (crates/backend/cuda-kernels/src/tile/attention/resident_attention_prefill_kernels.rs:378-469)
// and the CuTe-generated sm_100a artifact that the reference ships for another geometry only
// (crates/backend/cuda/kernels/fa4-attention/README.md:30-34).  Formula:
// crates/testing/cpu/reference-ops/src/kernels.rs:251-297.
#include <cuda.h>
#include <math.h>
#include <mutex>
#include <unordered_map>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

namespace {

constexpr int kRows = 128;             // rows of a CTA = MMA M
constexpr int kKeys = 128;             // keys per tile = MMA N of S, K extent of P V
// Threads: TMA warp, MMA warp, 8 softmax warps (two threads per row) per row block.
// K and V tiles in flight, by head size and row blocks per CTA (what shared memory holds beside
// Q; one block issues its scores two key tiles ahead, two blocks one tile ahead).
__host__ __device__ constexpr int stages_k(int d, int qb) { return qb == 2 ? (d == 128 ? 2 : 3) : 3; }   // scores run one (two blocks) or two tiles ahead
__host__ __device__ constexpr int stages_v(int d, int qb) { return d == 128 ? 2 : 3; }
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.0f;   // log2 units

// K-major operand (rows of 128 bytes along K, 8-row groups `group_bytes` apart), 128-byte swizzle.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr, uint32_t group_bytes = 1024) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)((group_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand: 128-byte rows run along MN (64 elements), one row per K index, 8 K
// indices per 1024-byte group, the groups `k_group_bytes` apart (stride byte offset); the next
// 64 MN elements are `mn_group_bytes` further (leading byte offset).  128-byte swizzle.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t mn_group_bytes, uint32_t k_group_bytes) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((mn_group_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((k_group_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// D 32-bit, A bfloat16 K-major, B bfloat16 K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int mma_m, int mma_n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(mma_n >> 3) << 17) |
         ((uint32_t)(mma_m >> 4) << 24);
}
__device__ __forceinline__ void tmem_store_32(uint32_t addr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(addr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_store_32u(uint32_t addr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(addr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 columns of this thread's lane into v[0..31]; the values may be used after tmem_wait_ld().
__device__ __forceinline__ void tmem_load_32_nowait(uint32_t addr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// D (tensor memory) (+)= A (tensor memory: row = lane, two bfloat16 of consecutive K per 32-bit
// column) * B (shared memory descriptor).
__device__ __forceinline__ void mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// 2^x by the special-function unit (2 ulp; the result is rounded to bfloat16 anyway).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Params {
  __nv_bfloat16* out;
  const int* positions; const int* cu_q; const int* block_table;
  int* error_flag;
  int max_blocks, n_seqs, nq, nkv, window, out_stride, page_size, num_pages;
  float scale_log2;
  int skip_single;       // sequences that bring one token are somebody else's (the decode kernel's)
};

// QB = row blocks of a CTA.  Measured on this part (one thread issuing, operands in place): a
// tcgen05.mma of 128 rows takes 104 clocks with both operands in shared memory and 87 with A
// in tensor memory whatever its N up to 128 (170 at N = 256), so a 128 x 128 score tile and
// its P V cost 8 x 107 + 8 x 87 = 1,550 clocks of the tensor core, and the exponentials
// 1,024 clocks of the special-function unit (16 a clock and SM).
//   One block: its scores alternate between two S buffers and are issued two tiles ahead, so
//   the softmax warps never wait for the tensor core; a tile takes as long as their loop.
//   Two blocks (256 rows, consecutive tokens of one sequence; for long prompts): they share
//   every K and V tile that comes in; tensor memory holds one S buffer and O per block (4 x
//   128 columns), scores are issued one tile ahead, and while one block's warps work on a
//   tile the tensor core works for the other block.
template <int D, int QB>
__global__ void __launch_bounds__(64 + 256 * QB)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k_run,
                  const __grid_constant__ CUtensorMap map_v_run, const Params p) {
  constexpr int kChunks = D / 64;                       // 64-wide slices of the head
  constexpr uint32_t kSlice = kRows * 128;              // bytes of a [128][64] bf16 slice
  constexpr uint32_t kQBytes = kChunks * kSlice;        // one row block of Q
  // A K or V tile lies as [group of 8 keys][slice of the head][8 keys][64]: a page of the
  // cache, whole, is one TMA box (key in group, slice, group in page are dimensions of the
  // tensor map), and so is a run of pages that follow one another in the pool.  (With one box
  // per page and slice, pages scattered over the pool cost 32 boxes of 2 KB per tile of K and
  // V, and the TMA unit takes ≈26 ns per box whatever its size: 512 tokens behind 3,584 took
  // 72 us against 48 us with the pages in order; whole pages: 58 us.  In order this layout is
  // 2 % slower than slice-major tiles were; choosing between the two per stage cost the
  // issuing thread more than that.)
  constexpr uint32_t kKBytes = kChunks * kSlice;
  constexpr uint32_t kVBytes = kChunks * kSlice;
  constexpr uint32_t kGroup = kChunks * 1024;           // bytes from one group of 8 keys to the next
  constexpr int kStagesK = stages_k(D, QB), kStagesV = stages_v(D, QB);
  constexpr int KS = kKeys;                             // keys of a score tile
  constexpr int SUB = kKeys / KS;                       // score tiles per K / V tile
  constexpr int NBUF = QB == 2 ? 1 : 2;                 // S buffers per block = score tiles issued ahead
  constexpr int E = KS / 2;                             // scores per softmax thread and score tile
  constexpr uint32_t kTmemCols = 512;                   // S buffers: QB x NBUF x 128 columns = 256; then O of each block: 128 columns apart
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();                      // q, the cache and the step's arrays come from earlier work in the stream

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base, k_s = q_s + QB * kQBytes, v_s = k_s + kStagesK * kKBytes, end_s = v_s + kStagesV * kVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (end_s - base));
  const uint32_t bar0 = smem_u32(bars);
  // s_full[t], p_full[t]: S tile t holds scores / holds the probabilities made from them;
  // o_done[q]: the last O += P V of block q that was issued has run
  const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = k_full + 8 * kStagesK, v_full = k_empty + 8 * kStagesK,
                 v_empty = v_full + 8 * kStagesV, s_full = v_empty + 8 * kStagesV, p_full = s_full + 32, o_done = p_full + 32;
  constexpr int kBars = 1 + 2 * kStagesK + 2 * kStagesV + 10;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + kBars);
  volatile int* failed = reinterpret_cast<volatile int*>(bars + kBars + 1);
  float* xmax_all = reinterpret_cast<float*>(bars + kBars + 2);      // per block: [2][2][128] row maxima, then [2][128] row sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.nq / p.nkv;
  const int kvh = blockIdx.x;           // heads vary fastest, so that the longest runs of every head start first
  const int tokens_per_block = kRows / G;
  const int tokens_per_cta = QB * tokens_per_block;

  // which sequence and which run of its tokens; the runs with the most keys first
  int seq = 0, tile = (int)gridDim.y - 1 - (int)blockIdx.y;
  for (; seq < p.n_seqs; ++seq) {
    const int n = p.cu_q[seq + 1] - p.cu_q[seq];
    const int tiles = (p.skip_single && n == 1) ? 0 : (n + tokens_per_cta - 1) / tokens_per_cta;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (seq >= p.n_seqs) return;
  const int tok0 = p.cu_q[seq], q_len = p.cu_q[seq + 1] - tok0;
  const int t_first = tile * tokens_per_cta;
  const int t_last = min(q_len, t_first + tokens_per_cta) - 1;
  // positions are written by the step's staging copy, an earlier operation in the stream
  const int pos_first = p.positions[tok0 + t_first], pos_last = p.positions[tok0 + t_last];
  const int key_lo = (p.window > 0 && pos_first + 1 > p.window) ? pos_first + 1 - p.window : 0;
  const int first_tile = key_lo / kKeys;
  const int n_tiles = pos_last / kKeys - first_tile + 1;      // both blocks walk all of them; what a row may not see is masked
  const int* table = p.block_table + (size_t)seq * p.max_blocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStagesK; ++s) { mbar_init(k_full + 8 * s, 1); mbar_init(k_empty + 8 * s, 1); }
    for (int s = 0; s < kStagesV; ++s) { mbar_init(v_full + 8 * s, 1); mbar_init(v_empty + 8 * s, 1); }
    for (int t = 0; t < 4; ++t) { mbar_init(s_full + 8 * t, 1); mbar_init(p_full + 8 * t, 256); }
    for (int t = 0; t < 2; ++t) mbar_init(o_done + 8 * t, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);      // (the same in every lane, and known to be)
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 256;
  // Score tile u of block q goes to S buffer NBUF q + u % NBUF, and this is use u / NBUF of
  // it; the barrier pairs s_full / p_full are indexed like the buffers.
  const int n_sub = n_tiles * SUB;
  auto s_buf = [](int q, int u) { return NBUF * q + (u % NBUF); };
  auto s_use = [](int u) { return u / NBUF; };
  auto s_cols = [&](int q, int u) { return tmem_s + (uint32_t)(s_buf(q, u) * KS); };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // A tile is up to 16 boxes per tensor (one per page and 64-wide slice of the head); the
    // warp's lanes issue them side by side, lanes 0-15 the K boxes and 16-31 the V boxes,
    // after lane 0 has seen the stage free and armed its barrier.
    if (lane == 0) {
      // a block's box is G heads x tokens_per_block tokens: that many rows of 128 bytes per slice
      mbar_expect_tx(q_full, (uint32_t)(QB * kChunks * tokens_per_block * G * 128));
#pragma unroll
      for (int q = 0; q < QB; ++q)
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(q_s + q * kQBytes + c * kSlice, &map_q, q_full, c * 64, kvh * G, tok0 + t_first + q * tokens_per_block);
    }
    const int pages_per_tile = kKeys / p.page_size;
    const int box_page = lane & 15;                       // lanes 0-15 bring K pages, 16-31 V pages
    const bool has_box = box_page < pages_per_tile;
    const uint32_t page_bytes = (uint32_t)p.page_size * D * 2;
    const int groups_per_page = p.page_size / 8;
    const int run_boxes = pages_per_tile > 1 ? 2 : 1;     // a run of pages comes as two boxes side by side (one, if the tile is one page)

    bool ok = true;
    auto lookup = [&](int j) {                            // page of this lane's box of tile j
      int page = p.num_pages;                             // outside the tensor: TMA fills zeros
      if (has_box && j < n_tiles) {
        const int key0 = (first_tile + j) * kKeys;
        const int blk = key0 / p.page_size + box_page;
        const int pg = blk < p.max_blocks ? __ldg(table + blk) : -1;
        if (pg >= 0 && pg < p.num_pages && key0 + box_page * p.page_size <= pos_last) page = pg;
      }
      return page;
    };
    // The K ring and the V ring are filled independently, each as soon as it has a free stage
    // (scores run ahead of the products that free V stages, so K tiles are wanted earlier).
    // The TMA unit takes tens of nanoseconds per box whatever its size: a box is a whole page
    // (up to 8 boxes of 4 KB per tile and tensor), or, when the tile's pages follow one another
    // in the pool (pages are handed out in order), half the tile.
    int jk = 0, jv = 0;
    int page_k = lookup(0), page_v = page_k;               // pages of this lane's box of tiles jk and jv
    uint32_t idle = 0;
    while ((jk < n_tiles || jv < n_tiles) && ok) {
      int free_k = 0, free_v = 0;
      if (lane == 0) {
        free_k = jk < n_tiles && (jk < kStagesK || mbar_test_wait(k_empty + 8 * (jk % kStagesK), ((jk / kStagesK) - 1) & 1));
        free_v = jv < n_tiles && (jv < kStagesV || mbar_test_wait(v_empty + 8 * (jv % kStagesV), ((jv / kStagesV) - 1) & 1));
      }
      free_k = __shfl_sync(0xffffffffu, free_k, 0);
      free_v = __shfl_sync(0xffffffffu, free_v, 0);
      if (free_k) {
        const int s = jk % kStagesK;
        const int page = page_k;
        page_k = lookup(jk + 1);                            // in flight while this tile's boxes are issued
        const int first_page = __shfl_sync(0xffffffffu, page, 0);
        const bool run = __all_sync(0xffffffffu, !has_box || page == first_page + box_page) &&
                         first_page + pages_per_tile <= p.num_pages;
        if (lane == 0) mbar_expect_tx(k_full + 8 * s, kKBytes);
        __syncwarp();
        if (run) {
          if (lane < run_boxes)
            tma_load_5d(k_s + s * kKBytes + lane * (kKBytes / 2), &map_k_run, k_full + 8 * s, 0, 0, 0, kvh * groups_per_page,
                        first_page + lane * (pages_per_tile / 2));
        } else if (has_box && lane < 16)
          tma_load_5d(k_s + s * kKBytes + box_page * page_bytes, &map_k, k_full + 8 * s, 0, 0, 0, 0, page * p.nkv + kvh);
        ++jk;
      }
      if (free_v) {
        const int sv = jv % kStagesV;
        const int page = page_v;
        page_v = lookup(jv + 1);
        const int first_page = __shfl_sync(0xffffffffu, page, 0);
        const bool run = __all_sync(0xffffffffu, !has_box || page == first_page + box_page) &&
                         first_page + pages_per_tile <= p.num_pages;
        if (lane == 0) mbar_expect_tx(v_full + 8 * sv, kVBytes);
        __syncwarp();
        if (run) {
          if (lane >= 16 && lane < 16 + run_boxes)
            tma_load_5d(v_s + sv * kVBytes + (lane - 16) * (kVBytes / 2), &map_v_run, v_full + 8 * sv, 0, 0, 0, kvh * groups_per_page,
                        first_page + (lane - 16) * (pages_per_tile / 2));
        } else if (has_box && lane >= 16)
          tma_load_5d(v_s + sv * kVBytes + box_page * page_bytes, &map_v, v_full + 8 * sv, 0, 0, 0, 0, page * p.nkv + kvh);
        ++jv;
      }
      if (free_k || free_v) idle = 0;
      else if (++idle > 64u * kWaitLimit) ok = false;       // bounded like every other wait (a poll here returns at once)
    }
    if (!ok && lane == 0) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // (One lane issues.  Having the whole warp walk this loop with lane 0 predicated, so that
    // the operands could stay in uniform registers, was measured and was slower.)
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(kRows, KS, 0);
      constexpr uint32_t idesc_o = instr_desc(kRows, D, 1);
      bool ok = mbar_wait(q_full, 0);
      // scores of (block q, score tile u) = Q_q K^T over the tile's KS keys, into their S buffer
      auto issue_s = [&](int q, int u) {
        const int j = u / SUB, h = u % SUB, s = j % kStagesK;
        ok = ok && mbar_wait(k_full + 8 * s, (j / kStagesK) & 1);
        if (!ok) return;
        tcgen05_fence_after();
        const uint32_t acc = s_cols(q, u);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_bf16(acc, desc_k_major(q_s + q * kQBytes + c * kSlice) + 2 * k,
                     desc_k_major(k_s + s * kKBytes + c * 1024 + h * (KS / 8) * kGroup, kGroup) + 2 * k, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(s_full + 8 * s_buf(q, u));
      };
      // The scores that next use an S buffer are issued right behind the O += P V that reads P
      // from it.  The tensor core executes what one thread issues in the order of issue, so
      // the product has read P before the new scores overwrite it; and P was only written
      // after the softmax warps had read the scores that were there.
      // K and V stages go back to the producer once every block has issued its last use of
      // them (a commit covers everything issued before it).
      int s_issued[QB], pv_issued[QB], k_released = 0, v_released = 0;
#pragma unroll
      for (int q = 0; q < QB; ++q) { s_issued[q] = 0; pv_issued[q] = 0; }
      auto release = [&]() {
        int s_min = s_issued[0], pv_min = pv_issued[0];
#pragma unroll
        for (int q = 1; q < QB; ++q) { s_min = min(s_min, s_issued[q]); pv_min = min(pv_min, pv_issued[q]); }
        for (; k_released < s_min / SUB; ++k_released) tcgen05_commit(k_empty + 8 * (k_released % kStagesK));
        for (; v_released < pv_min / SUB; ++v_released) tcgen05_commit(v_empty + 8 * (v_released % kStagesV));
      };
      for (int u = 0; u < NBUF && u < n_sub; ++u)
        for (int q = 0; q < QB && ok; ++q) { issue_s(q, u); s_issued[q] = u + 1; }
      release();
      // Whichever block has its probabilities ready is served next: the blocks drift apart by
      // half a tile and then take turns at the special-function unit and at the tensor core.
      int left = QB * n_sub;
      uint32_t idle = 0;
      while (left > 0 && ok) {
        bool any = false;
#pragma unroll
        for (int q = 0; q < QB; ++q) {
          const int u = pv_issued[q];
          if (u >= n_sub || !ok) continue;
          if (!mbar_test_wait(p_full + 8 * s_buf(q, u), s_use(u) & 1)) continue;
          const int j = u / SUB, h = u % SUB, sv = j % kStagesV;
          ok = ok && mbar_wait(v_full + 8 * sv, (j / kStagesV) & 1);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t p_t = s_cols(q, u);       // P: KS / 2 columns, two bfloat16 of consecutive keys each
#pragma unroll
          for (int k = 0; k < KS / 16; ++k)   // 16 keys a step: 8 columns of P, two 8-key groups of V
            mma_bf16_ts(tmem_o + (uint32_t)q * 128u, p_t + 8 * k, desc_mn_major(v_s + sv * kVBytes + (h * (KS / 16) + k) * 2 * kGroup, 1024, kGroup),
                        idesc_o, (u > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit(o_done + 8 * q);
          pv_issued[q] = u + 1;
          if (u + NBUF < n_sub) { issue_s(q, u + NBUF); s_issued[q] = u + NBUF + 1; }
          release();
          --left;
          any = true;
        }
        if (any) idle = 0;
        else if (++idle > 64u * kWaitLimit) ok = false;       // bounded like every other wait (a poll here returns at once)
      }
      if (!ok) {
        *failed = 1; if (p.error_flag) *p.error_flag = 1;
        for (int t = 0; t < 4; ++t) tcgen05_commit(s_full + 8 * t);          // let the softmax warps leave their waits
        tcgen05_commit(o_done); tcgen05_commit(o_done + 8);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax, correction, output
    // Per block eight warps, two threads per row: four warps take keys 0..63 of a tile (and the
    // first half of the head's columns of O), four take keys 64..127 (and the second half).
    const int q = (warp - 2) >> 3;                       // row block of this warp
    const int quad = warp & 3;
    const int half = ((warp - 2) & 7) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float* xmax = xmax_all + q * 768;
    const uint32_t o_t = tmem_o + (uint32_t)q * kKeys + lane_addr;
    const int tl = t_first + q * tokens_per_block + row / G;
    const bool live = row < tokens_per_block * G && tl < q_len;     // rows past the last whole token hold no query
    const int head = kvh * G + row % G;
    const int pos = live ? p.positions[tok0 + tl] : -1;
    const int lo = (live && p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
    constexpr int kOCols = D / 2;                      // columns of O this thread owns
    float m_used = -1e30f, l = 0.f;
    bool ok = true;
    auto block_sync = [&]() {                           // the 256 threads of this row block
      if (q == 0) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 2, 256;" ::: "memory");
    };
    for (int u = 0; u < n_sub; ++u) {
      const int key0 = first_tile * kKeys + u * KS + half * E;
      const int t = s_buf(q, u);
      const uint32_t s_t = s_cols(q, u) + lane_addr;     // this row of the S buffer
      // `ok` only ever changes through waits that all 256 threads of the block share, so they
      // leave the loop together and nobody is left alone at the named barrier below
      if (!mbar_wait(s_full + 8 * t, s_use(u) & 1)) ok = false;
      tcgen05_fence_after();
      if (!ok) break;
      float v[E];
#pragma unroll
      for (int c0 = 0; c0 < E; c0 += 32) tmem_load_32_nowait(s_t + half * E + c0, v + c0);
      tmem_wait_ld();
      // raw scores stay in v (the scale is positive and folds into the exponent's multiply-add);
      // keys this row may not see become -inf; the maximum is taken in log2 units, in four
      // chains so that no instruction waits for the one before it
      const bool all_visible = key0 + E - 1 <= pos && key0 >= lo;
      if (!all_visible) {
#pragma unroll
        for (int c = 0; c < E; ++c) {
          const int key = key0 + c;
          v[c] = (key <= pos && key >= lo) ? v[c] : -INFINITY;
        }
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < E; c += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) m4[i] = fmaxf(m4[i], v[c + i]);
      }
      float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      xmax[(u & 1) * 256 + half * 128 + row] = mx;
      // (this barrier also separates every thread's reads of S from the other half's writes of P below)
      block_sync();
      mx = fmaxf(mx, xmax[(u & 1) * 256 + (half ^ 1) * 128 + row]);
      const bool grow = mx > m_used + kRescaleStep;
      const float m_new = grow ? mx : m_used;
      // exponentials and the row sum (two chains); P as bfloat16, two keys to a 32-bit word
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t packed[E / 2];
#pragma unroll
      for (int e = 0; e < E / 2; ++e) {
        const float e0 = ex2(fmaf(v[2 * e], p.scale_log2, -m_new));
        const float e1 = ex2(fmaf(v[2 * e + 1], p.scale_log2, -m_new));
        sum0 += e0; sum1 += e1;
        __nv_bfloat162 hh = __floats2bfloat162_rn(e0, e1);
        packed[e] = *reinterpret_cast<uint32_t*>(&hh);
      }
      // O is at rest once the block's previous P V has run (it ran while the exponentials above
      // were taken; waiting for it every tile also keeps this thread's count of the barrier's phases exact)
      if (u > 0 && !mbar_wait(o_done + 8 * q, (u - 1) & 1)) ok = false;
      if (!ok) break;
      if (__any_sync(0xffffffffu, grow)) {
        const float corr = exp2f(m_used - m_new);
        if (u > 0) {
          tcgen05_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < kOCols; c0 += 32) {
            float o[32];
            tmem_load_32(o_t + half * kOCols + c0, o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= corr;
            tmem_store_32(o_t + half * kOCols + c0, o);
          }
        }
        l *= corr;
        m_used = m_new;
      }
      l += sum0 + sum1;
      // P takes the first KS / 2 columns of the S buffer its scores came from: this thread's
      // keys are columns (E / 2) half .. (E / 2) half + E / 2 - 1
      tmem_store_32u(s_t + half * (E / 2), packed);
      tcgen05_fence_before();
      mbar_arrive(p_full + 8 * t);
    }
    if (ok && !mbar_wait(o_done + 8 * q, (n_sub - 1) & 1)) ok = false;
    tcgen05_fence_after();
    if (!ok) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
    // the two halves of a row add their sums
    xmax[512 + half * 128 + row] = l;
    block_sync();
    l += xmax[512 + (half ^ 1) * 128 + row];
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t)(tok0 + (live ? tl : 0)) * p.out_stride + (size_t)head * D + half * kOCols;
#pragma unroll 1
      for (int c0 = 0; c0 < kOCols; c0 += 32) {
        float o[32];
        tmem_load_32(o_t + half * kOCols + c0, o);       // collective: every lane of the warp takes part
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(o[8 * g] * inv, o[8 * g + 1] * inv);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(o[8 * g + 2] * inv, o[8 * g + 3] * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[8 * g + 4] * inv, o[8 * g + 5] * inv);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(o[8 * g + 6] * inv, o[8 * g + 7] * inv);
            w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
            w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + c0 + 8 * g) = w;
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ host side
int encode(CUtensorMap* out, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
           const cuuint32_t* box, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail("attention (tensor cores): cuTensorMapEncodeTiled is not available from this driver");
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("attention (tensor cores): cuTensorMapEncodeTiled failed for %s with code %d", what, (int)r);
  return 0;
}

template <int D, int QB>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mkr,
           const CUtensorMap& mvr, const Params& p, int n_tiles, cudaStream_t stream) {
  constexpr int kChunks = D / 64;
  constexpr int kStagesK = stages_k(D, QB), kStagesV = stages_v(D, QB);
  constexpr size_t smem = (size_t)kChunks * kRows * 128 * (QB + kStagesK + kStagesV) + 1024 +
                          (1 + 2 * kStagesK + 2 * kStagesV + 10 + 2) * 8 + (size_t)QB * 768 * 4;
  static_assert(smem <= 227 * 1024, "tiles do not fit shared memory");
  static OncePerDevice once;
  if (once.first()) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<D, QB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) once.forget();
    if (e != cudaSuccess) return fail("attention (tensor cores): cannot reserve %zu bytes of shared memory", smem);
  }
  ilb::launch(prefill_tc_kernel<D, QB>, dim3(p.nkv, n_tiles), dim3(64 + 256 * QB), smem, stream, mq, mk, mv, mkr, mvr, p);
  return check_launch("attention prefill (tensor cores)");
}

}  // namespace

// Geometry this kernel is built for; everything else takes attention_flash / attention_simple.
ILB_EXPORT int ilb_attention_tc_supported(int nq, int nkv, int d, int page_size) {
  if (nkv <= 0 || nq % nkv != 0) return 0;
  const int g = nq / nkv;
  return ((d == 64 || d == 128) && g <= 128 &&
          (page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128)) ? 1 : 0;
}

// row_blocks = 1 or 2 blocks of 128 rows per CTA (two share every K and V tile: for long
// portions); n_tiles = sum over sequences of ceil(q_len / (row_blocks * floor(128 / G))),
// without the sequences of one token if skip_single is set (their rows of `out` are then
// left alone).
ILB_EXPORT int ilb_attention_prefill_tc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                        const int* positions, const int* cu_q, const int* block_table,
                                        int max_blocks, int page_size, int num_pages, int window, float scale,
                                        int n_tokens, int n_seqs, int n_tiles, int row_blocks, int skip_single, int nq, int nkv, int d,
                                        int q_stride, int out_stride, int* error_flag, cudaStream_t stream) {
  ILB_REQUIRE(row_blocks == 1 || row_blocks == 2, "attention (tensor cores): %d row blocks per CTA (1 or 2)", row_blocks);
  ILB_REQUIRE(ilb_attention_tc_supported(nq, nkv, d, page_size),
              "attention (tensor cores): heads %d/%d, head size %d, page size %d are not built", nq, nkv, d, page_size);
  ILB_REQUIRE(n_tokens > 0 && n_seqs > 0 && n_tiles > 0 && n_tiles <= 65535 && max_blocks > 0 && num_pages > 0 && window >= 0,
              "attention (tensor cores): bad sizes");
  ILB_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)q % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
              ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0), "attention (tensor cores): misaligned operands");
  const int G = nq / nkv;
  CUtensorMap mq, mk, mv, mkr, mvr;
  {   // q as (d, heads, tokens); a box is 64 x G x floor(128/G) = the rows of a tile, one slice of the head
    const cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)nq, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(kRows / G)};
    if (encode(&mq, q, 3, dims, strides, box, "q")) return -1;
  }
  {   // The cache [page][kv head][key][d] as (64 of d, key in its group of 8, slice of the head,
      // group in the page, page x kv head): a box is the whole page of one head and lands as
      // [group][slice][8 keys][64], the operand layout with its groups 1 or 2 KB apart.
      // (The strides are not ascending: the encoder takes that; the coordinates are all zero
      // but the last, so every copy starts on a 16-byte boundary.)
    const cuuint64_t slices = (cuuint64_t)d / 64, groups = (cuuint64_t)page_size / 8;
    const cuuint64_t dims[5] = {64, 8, slices, groups, (cuuint64_t)num_pages * nkv};
    const cuuint64_t strides[4] = {(cuuint64_t)d * 2, 128, (cuuint64_t)d * 2 * 8, (cuuint64_t)d * 2 * page_size};
    const cuuint32_t box[5] = {64, 8, (cuuint32_t)slices, (cuuint32_t)groups, 1};
    if (encode(&mk, k_cache, 5, dims, strides, box, "k cache")) return -1;
    if (encode(&mv, v_cache, 5, dims, strides, box, "v cache")) return -1;
    // the same with (group in the page, kv head) as one dimension and the page as the last: a
    // box spans half the pages of a 128-key tile when their numbers follow one another
    const cuuint64_t rdims[5] = {64, 8, slices, groups * nkv, (cuuint64_t)num_pages};
    const cuuint64_t rstrides[4] = {(cuuint64_t)d * 2, 128, (cuuint64_t)d * 2 * 8, (cuuint64_t)d * 2 * page_size * nkv};
    const int pages_per_tile = kKeys / page_size;
    const cuuint32_t run[5] = {64, 8, (cuuint32_t)slices, (cuuint32_t)groups, (cuuint32_t)(pages_per_tile > 1 ? pages_per_tile / 2 : 1)};
    if (encode(&mkr, k_cache, 5, rdims, rstrides, run, "k cache (page run)")) return -1;
    if (encode(&mvr, v_cache, 5, rdims, rstrides, run, "v cache (page run)")) return -1;
  }
  Params p{(__nv_bfloat16*)out, positions, cu_q, block_table, error_flag, max_blocks, n_seqs, nq, nkv, window,
           out_stride, page_size, num_pages, scale * kLog2e, skip_single ? 1 : 0};
  if (row_blocks == 2)
    return d == 64 ? launch<64, 2>(mq, mk, mv, mkr, mvr, p, n_tiles, stream) : launch<128, 2>(mq, mk, mv, mkr, mvr, p, n_tiles, stream);
  return d == 64 ? launch<64, 1>(mq, mk, mv, mkr, mvr, p, n_tiles, stream) : launch<128, 1>(mq, mk, mv, mkr, mvr, p, n_tiles, stream);
}

ILB_DEFINE_LAST_ERROR()
