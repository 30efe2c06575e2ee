// Split-KV decode attention over the paged bfloat16 cache: one token per sequence, the
// keys of a (sequence, kv head) shared out over the CTAs of a thread-block cluster, K and
// V tiles brought by TMA straight from the cache pages, the partial results merged through
// the cluster's shared memory.
//
//   grid     (S, kv heads, sequences x Z), clusters of S = 1..16 along x, S chosen so that all
//            CTAs of the launch are resident at once.  The visible keys are cut into 32-key
//            tiles; tile i goes to CTA i % S of the cluster.  Few sequences with many keys
//            (the caller says so): Z = 2..8 clusters share a (sequence, kv head), each taking a
//            contiguous run of its tiles, as many of them as the sequence's length calls for;
//            their merged records meet in a scratch buffer and the owner that takes the last
//            ticket of its rows adds them in the order of the runs (no CTA waits for another).
//   warp 2   producer: 8 lanes look up the pages of a tile (lookups of the next four tiles are
//            always in flight) and issue its boxes: K and V, each as one box per page part
//            and 64-wide slice of the head, 128-byte swizzle, into a ring of 3 to 12 stages guarded
//            by full/empty mbarriers.  A page that is not held is requested outside the tensor,
//            which TMA fills with zeros.
//   warps 0-1  consumers: the group's query heads are the 16 rows of an m16n8k16 MMA; each
//            warp takes 16 keys of every tile: S = Q K^T, online softmax in 32-bit, O += P V
//            with ldmatrix from the swizzled tiles.
//   merge    a group of up to 16 query heads: the two warps' (max, sum, O) become one record
//            in the CTA; row r of it is SENT to CTA r % S of the cluster (asynchronous stores
//            that count on the owner's mbarrier), and the owner adds the S records of its rows
//            in the order of the CTAs from its own shared memory.  One cluster barrier, at
//            the start (so that every mbarrier is ready); no scratch buffer, no tickets, no
//            second pass through L2.  Larger groups run in passes of 16 heads whose records
//            stay where they are and are read by the cluster between two barriers.
//   input    with the fused projection output as input, the consumers norm and rotate q on
//            the way into their MMA fragments, and the warp whose keys include the step's own
//            position norms and rotates the new key, writes it and the new value to the cache
//            and patches them into the tile in shared memory.  The producer warp then reads
//            nothing that the preceding kernel writes and starts its stream before the
//            dependency wait.
// Every mbarrier wait is bounded; on expiry a flag is raised and the CTA leaves (or, in the
// form with cluster barriers, still walks to them), so nobody is left waiting.  No multicast.
//
// Reference counterparts: `partial_gqa_lanes` + `merge_gqa`, split-KV decode with the
// group's heads padded to 16 MMA rows
// (crates/backend/cuda-kernels/src/tile/attention/resident_attention_decode_kernels.rs:
// 131-226, :417-451, :497-598).  Formula: crates/testing/cpu/reference-ops/src/kernels.rs:251-297.
#include <cuda.h>
#include <math.h>
#include <mutex>
#include <unordered_map>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

namespace {

constexpr int kKeys = 32;              // keys per tile
constexpr int kMaxSplit = 16;          // CTAs of a cluster: 1, 2, 4, 8 or 16
constexpr int kConsumers = 2;          // warps, 16 keys of a tile each
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kAhead = 4;              // tiles whose page lookups are in flight
constexpr int kChunkTiles = 8;         // tiles a CTA should have before another cluster joins its sequence
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  const __nv_bfloat16* q; __nv_bfloat16* out;
  const int* positions; const int* cu_q; const int* block_table;
  int* error_flag;
  int max_blocks, n_seqs, nq, nkv, window, q_stride, out_stride, page_size, num_pages;
  int split;                           // CTAs of a cluster = ways a sequence's tiles are dealt out
  int rows_cap;                        // rows of the group that one CTA of the cluster owns at most
  // Few sequences with many keys: `chunks` clusters share a (sequence, kv head), each taking a
  // contiguous run of its tiles (as many of them as leave kChunkTiles tiles to every CTA).
  // Their merged records meet in `scratch` [sequence][kv head][chunk][16][D + 2]; the owner
  // that takes the last ticket of its rows (`counters` [sequence][kv head][16], zero between
  // launches) adds them in chunk order and writes the result.
  int chunks; float* scratch; int* counters;
  float scale_log2;
  // Fused input stage (qkv != null): q, k, v of the step's token are taken from the fused
  // projection output; per-head RMSNorm (weights may be null) and the rotation (table may be
  // null) are applied here, the new key and value are written to the cache (unless the caches
  // to write are null) and patched into the tile that holds their position.
  const __nv_bfloat16* qkv; int qkv_stride;
  const float* q_weight; const float* k_weight; float eps;
  const float2* rope;                  // [tokens][D / 2] (cos, sin), rotation over the whole head
  __nv_bfloat16* k_write; __nv_bfloat16* v_write;
};

// Address of the 16-byte piece `chunk` (0..7) of row `row` in a [rows][128 bytes] slice
// written by TMA with the 128-byte swizzle (the slice starts on a 1024-byte boundary).
__device__ __forceinline__ uint32_t swz(uint32_t slice, int row, int chunk) {
  return slice + (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// 16 rows (query heads) of one warp: thread (g = lane / 4, t = lane % 4) owns rows g and
// g + 8, columns 2t, 2t + 1 of every 8-wide block.
template <int D>
struct RowState {
  float o[D / 8][4];
  float m[2], l[2];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

// 16 keys (rows row0 .. row0 + 15 of the tile's K and V slices, the first being key
// `key0`) against the warp's 16 query rows.  live[r]: row g + 8r is a head of the group;
// keys outside [lo, hi) are not seen.
template <int D>
__device__ __forceinline__ void tile_step(RowState<D>& st, const uint32_t (&q)[D / 16][4], uint32_t ks, uint32_t vs,
                                          int row0, int key0, const bool (&live)[2], int lo, int hi, float scale_log2,
                                          int lane) {
  constexpr uint32_t kSlice = kKeys * 128;           // bytes of one 64-wide slice of a tile
  const int t = lane & 3;
  float s[2][4];
#pragma unroll
  for (int nb = 0; nb < 2; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nb][e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; kk += 2) {
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      uint32_t r0, r1, r2, r3;
      const int col = kk * 16 + (lane >> 3) * 8;       // element of the head
      ldmatrix_x4(swz(ks + (col >> 6) * kSlice, row0 + nb * 8 + (lane & 7), (col & 63) >> 3), r0, r1, r2, r3);
      mma_16816(s[nb], q[kk], r0, r1);
      mma_16816(s[nb], q[kk + 1], r2, r3);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < 2; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + nb * 8 + 2 * t + (e & 1);
      const int r = e >> 1;
      const bool ok = live[r] && key >= lo && key < hi;
      s[nb][e] = ok ? s[nb][e] * scale_log2 : -INFINITY;
      mx[r] = fmaxf(mx[r], s[nb][e]);
    }
  float corr[2], base[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(st.m[r], mx[r]);
    base[r] = (m_new == -INFINITY) ? 0.f : m_new;
    corr[r] = exp2f(st.m[r] - base[r]);           // -inf -> 0
    st.m[r] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nb = 0; nb < 2; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float p = exp2f(s[nb][e] - base[e >> 1]);
      s[nb][e] = p;
      sum[e >> 1] += p;
    }
#pragma unroll
  for (int r = 0; r < 2; ++r) st.l[r] = st.l[r] * corr[r] + sum[r];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    st.o[i][0] *= corr[0]; st.o[i][1] *= corr[0];
    st.o[i][2] *= corr[1]; st.o[i][3] *= corr[1];
  }
  uint32_t a[4];
  a[0] = pack_bf16(s[0][0], s[0][1]);
  a[1] = pack_bf16(s[0][2], s[0][3]);
  a[2] = pack_bf16(s[1][0], s[1][1]);
  a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
  for (int nd = 0; nd < D / 16; ++nd) {
    uint32_t r0, r1, r2, r3;
    const int col = nd * 16 + (lane >> 4) * 8;
    ldmatrix_x4_trans(swz(vs + (col >> 6) * kSlice, row0 + (lane & 7) + ((lane >> 3) & 1) * 8, (col & 63) >> 3), r0, r1, r2, r3);
    mma_16816(st.o[2 * nd], a, r0, r1);
    mma_16816(st.o[2 * nd + 1], a, r2, r3);
  }
}

// Rows g and g + 8 of the warp's query heads from the fused projection output, as A
// fragments: per-head RMSNorm in 32-bit (sum over the row's four threads), then the rotation
// of pairs (i, i + D/2), which a thread holds both members of; rounded to bfloat16 once.
template <int D>
__device__ __forceinline__ void load_q_fused(uint32_t (&q)[D / 16][4], const __nv_bfloat16* row0, const __nv_bfloat16* row1,
                                             const float* weight, float eps, const float2* cs, int lane) {
  const int t = lane & 3;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const __nv_bfloat16* row = r == 0 ? row0 : row1;
    float x[D / 16][4];                                  // [kk][c, c+1, c+8, c+9], c = 16 kk + 2 t
    float ss = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int c = kk * 16 + 2 * t;
      __nv_bfloat162 a = __floats2bfloat162_rn(0.f, 0.f), b = a;
      if (row) {
        a = *reinterpret_cast<const __nv_bfloat162*>(row + c);
        b = *reinterpret_cast<const __nv_bfloat162*>(row + c + 8);
      }
      x[kk][0] = __low2float(a); x[kk][1] = __high2float(a); x[kk][2] = __low2float(b); x[kk][3] = __high2float(b);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss = fmaf(x[kk][e], x[kk][e], ss);
    }
    if (weight != nullptr) {
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int c = kk * 16 + 2 * t;
        x[kk][0] = x[kk][0] * inv * __ldg(weight + c);     x[kk][1] = x[kk][1] * inv * __ldg(weight + c + 1);
        x[kk][2] = x[kk][2] * inv * __ldg(weight + c + 8); x[kk][3] = x[kk][3] * inv * __ldg(weight + c + 9);
      }
    }
    if (cs != nullptr) {
#pragma unroll
      for (int kk = 0; kk < D / 32; ++kk) {                // column i < D/2 pairs with i + D/2 = block kk + D/32
        const int c = kk * 16 + 2 * t;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = c + (e & 1) + (e >> 1) * 8;
          const float2 w = __ldg(cs + i);
          const float a = x[kk][e], b = x[kk + D / 32][e];
          // products and sums rounded separately, as the reference's scalar code does
          x[kk][e] = __fsub_rn(__fmul_rn(a, w.x), __fmul_rn(b, w.y));
          x[kk + D / 32][e] = __fadd_rn(__fmul_rn(a, w.y), __fmul_rn(b, w.x));
        }
      }
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      q[kk][r] = row ? pack_bf16(x[kk][0], x[kk][1]) : 0u;
      q[kk][2 + r] = row ? pack_bf16(x[kk][2], x[kk][3]) : 0u;
    }
  }
}

// The step's own key and value (row `r` of a tile whose K slices start at `ks`, V slices at
// `vs`): normed and rotated key, raw value, written over what TMA brought for that row, and
// to the cache at `k_dst` / `v_dst` if those are not null.  Lane l holds elements
// E l .. E l + E - 1 of each half of the head (E = D / 64), the members of its rotation pairs.
template <int D>
__device__ __forceinline__ void patch_new_key(uint32_t ks, uint32_t vs, int r, const __nv_bfloat16* k_src,
                                              const __nv_bfloat16* v_src, const float* k_weight, float eps, const float2* cs,
                                              __nv_bfloat16* k_dst, __nv_bfloat16* v_dst, int lane) {
  constexpr int E = D / 64;
  constexpr uint32_t kSlice = kKeys * 128;
  float k[2][E], v[2][E];
  float ss = 0.f;
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const int e = h * (D / 2) + E * lane + i;
      k[h][i] = __bfloat162float(k_src[e]);
      v[h][i] = __bfloat162float(v_src[e]);
      ss = fmaf(k[h][i], k[h][i], ss);
    }
  if (k_weight != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < E; ++i) k[h][i] = k[h][i] * inv * __ldg(k_weight + h * (D / 2) + E * lane + i);
  }
  if (cs != nullptr) {
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const float2 w = __ldg(cs + E * lane + i);
      const float a = k[0][i], b = k[1][i];
      k[0][i] = __fsub_rn(__fmul_rn(a, w.x), __fmul_rn(b, w.y));
      k[1][i] = __fadd_rn(__fmul_rn(a, w.y), __fmul_rn(b, w.x));
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const int e = h * (D / 2) + E * lane + i;
      const __nv_bfloat16 kb = __float2bfloat16_rn(k[h][i]), vb = __float2bfloat16_rn(v[h][i]);
      const uint32_t off = (uint32_t)(e >> 6) * kSlice + (uint32_t)r * 128u +
                           (uint32_t)(((((e & 63) * 2) >> 4) ^ (r & 7)) << 4) + (uint32_t)(((e & 63) * 2) & 15);
      asm volatile("st.shared.b16 [%0], %1;" ::"r"(ks + off), "h"(*reinterpret_cast<const unsigned short*>(&kb)) : "memory");
      asm volatile("st.shared.b16 [%0], %1;" ::"r"(vs + off), "h"(*reinterpret_cast<const unsigned short*>(&vb)) : "memory");
      if (k_dst != nullptr) { k_dst[e] = kb; v_dst[e] = vb; }
    }
  __syncwarp();
}

template <int D, int kStages>
__global__ void __launch_bounds__(kThreads)
decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_k_run, const __grid_constant__ CUtensorMap map_v_run, const Params p) {
  constexpr int kSlices = D / 64;
  constexpr uint32_t kSlice = kKeys * 128;                 // bytes: one slice of one tensor of a tile
  constexpr uint32_t kTensor = kSlices * kSlice;           // K (or V) of a tile
  constexpr uint32_t kStage = 2 * kTensor;
  constexpr int kRec = D + 2;                              // O row, then max and sum
  static_assert(kConsumers * 16 * kRec * 4 <= kStages * (int)kStage, "records must fit the tile ring");

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - smem_u32(smem_raw));
  float* rec = reinterpret_cast<float*>(smem);             // [consumers][16][D + 2], once the tiles are consumed
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStage);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kStages;
  volatile int* failed = reinterpret_cast<volatile int*>(bars + 2 * kStages);
  // Records that the cluster sends here: [source CTA][row of this CTA][D + 4] (O, max, sum)
  constexpr int kRecIn = D + 4;
  const uint32_t inbox_bar = smem_u32(bars + 2 * kStages + 1);
  float* inbox = reinterpret_cast<float*>(bars + 2 * kStages + 2);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A group of at most 16 query heads (one pass) over a cluster: CTA r OWNS rows r, r + S, ...
  // of the group; every warp sends each row of its record to the row's owner, and an owner
  // waits only for the bytes of its rows.  Larger groups keep the form in which records stay
  // where they are and the cluster reads them between two barriers.
  const bool push = p.split > 1 && p.nq / p.nkv <= 16;
  const int rows_cap = p.rows_cap;                         // rows an owner holds at most (push)
  int rows_mine = 0;
  if (push) {
    const int G0 = p.nq / p.nkv, r0 = (int)blockIdx.x;
    rows_mine = G0 > r0 ? (G0 - r0 + p.split - 1) / p.split : 0;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, kConsumers); }
    if (push) mbar_init(inbox_bar, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (push && rows_mine > 0) mbar_expect_tx(inbox_bar, (uint32_t)(rows_mine * p.split * (D * 4 + 8)));
  }
  if (push) cluster_sync_all();          // every owner's mbarrier is ready before anything is sent to it
  else __syncthreads();
  // The step's positions and block tables were on the device before the step's first kernel
  // began, and the cache rows of earlier positions are older still.  When this kernel is the
  // one that writes the new position's key and value, nothing the producer warp reads comes
  // from the preceding kernel: it starts the stream of tiles without waiting for it.  Everyone
  // else reads the projection output and waits.
  const bool stream_early = p.qkv != nullptr && p.k_write != nullptr;
  if (!(stream_early && (threadIdx.x >> 5) == kConsumers)) pdl_wait();

  const int G = p.nq / p.nkv;
  const int rank = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z / p.chunks, chunk = blockIdx.z % p.chunks;
  const int tok = p.cu_q[seq];
  if (p.cu_q[seq + 1] - tok != 1) return;                  // the whole cluster leaves together
  const int pos = p.positions[tok];
  const int lo = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
  const int hi = pos + 1;
  const int kSplit = p.split;
  const int all_tiles = (hi + kKeys - 1) / kKeys - lo / kKeys;
  // the clusters that take part for this sequence, and this one's run of tiles
  int chunks_on = all_tiles / (kSplit * kChunkTiles);
  chunks_on = chunks_on < 1 ? 1 : (chunks_on > p.chunks ? p.chunks : chunks_on);
  if (chunk >= chunks_on) return;                          // (the whole cluster: nothing has been sent yet)
  const int per_chunk = (all_tiles + chunks_on - 1) / chunks_on;
  const int first_tile = lo / kKeys + chunk * per_chunk;
  const int n_tiles = min(per_chunk, all_tiles - chunk * per_chunk);
  const int n_my = rank < n_tiles ? (n_tiles - rank + kSplit - 1) / kSplit : 0;
  const int* table = p.block_table + (size_t)seq * p.max_blocks;
  const int rows16 = (G + 15) / 16 * 16;
  const int n_passes = rows16 / 16;
  auto key_of = [&](int j) { return (first_tile + rank + j * kSplit) * kKeys; };

  for (int pass = 0; pass < n_passes; ++pass) {            // 16 query heads of the group at a time
    const int rb = pass * 16;
    const int it0 = pass * n_my;                           // tiles this CTA has streamed in earlier passes
    if (warp == kConsumers) {
      // ------------------------------------------------------------ producer
      const int box_keys = p.page_size < kKeys ? p.page_size : kKeys;
      const int parts = kKeys / box_keys;
      const int per_tensor = kSlices * parts;
      const int b = lane;
      const bool has_box = b < 2 * per_tensor;
      const int which = b / per_tensor, rem = b % per_tensor, slice = rem / parts, part = rem % parts;
      auto lookup = [&](int j) {                           // page of this lane's box of tile j, or one past the tensor
        int page = p.num_pages;
        if (has_box && j < n_my) {
          const int key = key_of(j) + part * box_keys;
          const int blk = key / p.page_size;
          if (key < hi && blk < p.max_blocks) {
            const int pg = __ldg(table + blk);
            if (pg >= 0 && pg < p.num_pages) page = pg;
          }
        }
        return page;
      };
      int pg[kAhead];
#pragma unroll
      for (int i = 0; i < kAhead; ++i) pg[i] = lookup(i);
      bool ok = true;
      for (int j0 = 0; j0 < n_my && ok; j0 += kAhead) {
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          const int j = j0 + i;
          if (j >= n_my || !ok) break;
          const int it = it0 + j, s = it % kStages;
          if (lane == 0) {
            if (it >= kStages) ok = mbar_wait(empty0 + 8 * s, ((it / kStages) - 1) & 1);
            if (ok) mbar_expect_tx(full0 + 8 * s, kStage);
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          // The TMA unit's time per box hardly depends on its size: two 16-key pages that
          // follow one another in the pool come as one box.
          const int page_nb = __shfl_down_sync(0xffffffffu, pg[i], 1);
          const bool run = has_box && parts == 2 && part == 0 && pg[i] + 1 < p.num_pages && page_nb == pg[i] + 1;
          const bool covered = __shfl_up_sync(0xffffffffu, run ? 1 : 0, 1) != 0 && part == 1;
          if (run)
            tma_load_4d(base + s * kStage + which * kTensor + slice * kSlice, which == 0 ? &map_k_run : &map_v_run,
                        full0 + 8 * s, slice * 64, 0, kvh, pg[i]);
          else if (has_box && !covered)
            tma_load_4d(base + s * kStage + which * kTensor + slice * kSlice + part * box_keys * 128,
                        which == 0 ? &map_k : &map_v, full0 + 8 * s, slice * 64, (key_of(j) + part * box_keys) % p.page_size,
                        kvh, pg[i]);
          pg[i] = lookup(j + kAhead);
        }
      }
      if (!ok && lane == 0) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
    } else {
      // ------------------------------------------------------------ consumers
      const int g = lane >> 2, t = lane & 3;
      RowState<D> st;
      st.init();
      bool live[2];
      uint32_t q[D / 16][4];
#pragma unroll
      for (int r = 0; r < 2; ++r) live[r] = rb + g + 8 * r < G;
      if (p.qkv != nullptr) {
        const __nv_bfloat16* base_q = p.qkv + (size_t)tok * p.qkv_stride + (size_t)(kvh * G + rb) * D;
        load_q_fused<D>(q, live[0] ? base_q + (size_t)g * D : nullptr, live[1] ? base_q + (size_t)(g + 8) * D : nullptr,
                        p.q_weight, p.eps, p.rope ? p.rope + (size_t)tok * (D / 2) : nullptr, lane);
      } else {
        const __nv_bfloat16* row0 = live[0] ? p.q + (size_t)tok * p.q_stride + (size_t)(kvh * G + rb + g) * D : nullptr;
        const __nv_bfloat16* row1 = live[1] ? p.q + (size_t)tok * p.q_stride + (size_t)(kvh * G + rb + g + 8) * D : nullptr;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int c = kk * 16 + 2 * t;
          q[kk][0] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c) : 0u;
          q[kk][1] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c) : 0u;
          q[kk][2] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c + 8) : 0u;
          q[kk][3] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c + 8) : 0u;
        }
      }
      bool ok = true;
      for (int j = 0; j < n_my && ok; ++j) {
        const int it = it0 + j, s = it % kStages;
        ok = mbar_wait(full0 + 8 * s, (it / kStages) & 1);
        if (!ok) break;
        const int key0 = key_of(j) + warp * 16;
        if (p.qkv != nullptr && p.k_write != nullptr && pos >= key0 && pos < key0 + 16) {
          // this warp's slice of this tile holds the step's own position: its key and value
          // are not in the cache yet (the tile came with whatever the page held there)
          const __nv_bfloat16* row = p.qkv + (size_t)tok * p.qkv_stride;
          const int blk = pos / p.page_size;
          const int pg = blk < p.max_blocks ? __ldg(table + blk) : -1;
          const bool store = pass == 0 && pg >= 0 && pg < p.num_pages;     // never write outside the pool
          const size_t at = store ? (((size_t)pg * p.nkv + kvh) * p.page_size + (pos % p.page_size)) * D : 0;
          patch_new_key<D>(base + s * kStage, base + s * kStage + kTensor, pos % kKeys,
                           row + (size_t)(p.nq + kvh) * D, row + (size_t)(p.nq + p.nkv + kvh) * D, p.k_weight, p.eps,
                           p.rope ? p.rope + (size_t)tok * (D / 2) : nullptr, store ? p.k_write + at : nullptr,
                           store ? p.v_write + at : nullptr, lane);
          // TMA will write this stage again later: order these ordinary stores before it
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        if (key0 < hi)
          tile_step<D>(st, q, base + s * kStage, base + s * kStage + kTensor, warp * 16, key0, live, lo, hi, p.scale_log2, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);
      }
      if (!ok && lane == 0) { *failed = 1; if (p.error_flag) *p.error_flag = 1; }
      __syncwarp();
      if (push) {
        // The two warps' records become one (in the order warp 0, warp 1): warp 1 leaves its
        // fragments in the ring, lane by lane, once both warps are past their last tile.
        float l2[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          float l = st.l[r];
          l += __shfl_xor_sync(0xffffffffu, l, 1);
          l += __shfl_xor_sync(0xffffffffu, l, 2);
          l2[r] = l;
        }
        constexpr int kDump = D / 2 + 4;                     // floats a lane leaves: O fragments, two maxima, two sums
        float* dump = reinterpret_cast<float*>(smem);        // [kDump][32]
        static_assert(kDump * 32 * 4 <= kStages * (int)kStage, "a warp's fragments must fit the tile ring");
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
        if (warp == 1) {
#pragma unroll
          for (int i = 0; i < D / 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) dump[(i * 4 + c) * 32 + lane] = st.o[i][c];
#pragma unroll
          for (int r = 0; r < 2; ++r) { dump[(D / 2 + r) * 32 + lane] = st.m[r]; dump[(D / 2 + 2 + r) * 32 + lane] = l2[r]; }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
        if (warp == 0) {
          float f0[2], f1[2];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const float m1 = dump[(D / 2 + r) * 32 + lane], l1 = dump[(D / 2 + 2 + r) * 32 + lane];
            const float m = fmaxf(st.m[r], m1);
            f0[r] = st.m[r] == -INFINITY ? 0.f : exp2f(st.m[r] - m);
            f1[r] = m1 == -INFINITY ? 0.f : exp2f(m1 - m);
            st.m[r] = m;
            l2[r] = l2[r] * f0[r] + l1 * f1[r];
          }
#pragma unroll
          for (int i = 0; i < D / 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) st.o[i][c] = st.o[i][c] * f0[c >> 1] + dump[(i * 4 + c) * 32 + lane] * f1[c >> 1];
          // Row g + 8r goes to CTA (row % S), place row / S.  A lane holds pairs of columns;
          // neighbours of a quad trade one pair so that each sends 16 bytes at a time.
          const uint32_t me = (uint32_t)rank;
          const bool odd = (t & 1) != 0;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
            const uint32_t owner = (uint32_t)(row % kSplit);
            const uint32_t at = smem_u32(inbox) + 4u * (uint32_t)((me * rows_cap + row / kSplit) * kRecIn);
            const uint32_t dst = peer_addr(at, owner), bar = peer_addr(inbox_bar, owner);
#pragma unroll
            for (int i0 = 0; i0 < D / 8; i0 += 2) {
              const float ax = st.o[i0][2 * r], ay = st.o[i0][2 * r + 1], bx = st.o[i0 + 1][2 * r], by = st.o[i0 + 1][2 * r + 1];
              const float rx = __shfl_xor_sync(0xffffffffu, odd ? ax : bx, 1), ry = __shfl_xor_sync(0xffffffffu, odd ? ay : by, 1);
              if (live[r]) {
                if (!odd) st_peer_v4(dst + 4u * (uint32_t)(i0 * 8 + 2 * t), bar, ax, ay, rx, ry);
                else st_peer_v4(dst + 4u * (uint32_t)((i0 + 1) * 8 + 2 * (t - 1)), bar, rx, ry, bx, by);
              }
            }
            if (live[r] && t == 0) st_peer_v2(dst + 4u * (uint32_t)D, bar, st.m[r], l2[r]);
          }
        }
      } else {
      // both consumer warps are past their last tile before a record overwrites the ring
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumers * 32) : "memory");
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        float* row = rec + ((size_t)warp * 16 + g + 8 * r) * kRec;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { row[i * 8 + 2 * t] = st.o[i][2 * r]; row[i * 8 + 2 * t + 1] = st.o[i][2 * r + 1]; }
        if (t == 0) { row[D] = st.m[r]; row[D + 1] = l; }
      }
      }
    }
    if (push) {
      // ---- merge of the rows this CTA owns, from its own shared memory, CTA after CTA
      if (rows_mine > 0) {
        if (!mbar_wait(inbox_bar, 0)) { *failed = 1; if (p.error_flag) *p.error_flag = 1; return; }
        const int n_rec = kSplit;
        for (int e = threadIdx.x; e < rows_mine * D; e += kThreads) {
          const int slot = e / D, c = e % D, row = slot * kSplit + rank;
          const float* first = inbox + (size_t)slot * kRecIn;
          float m_all = -INFINITY;
          for (int i = 0; i < n_rec; ++i) m_all = fmaxf(m_all, first[(size_t)i * rows_cap * kRecIn + D]);
          float l_all = 0.f, o = 0.f;
          for (int i = 0; i < n_rec; ++i) {
            const float* rcd = first + (size_t)i * rows_cap * kRecIn;
            const float m = rcd[D];
            const float f = (m == -INFINITY) ? 0.f : exp2f(m - m_all);
            l_all += rcd[D + 1] * f;
            o += rcd[c] * f;
          }
          if (chunks_on == 1) {
            p.out[(size_t)tok * p.out_stride + (size_t)(kvh * G + row) * D + c] = __float2bfloat16_rn(l_all > 0.f ? o / l_all : 0.f);
          } else {
            // this cluster's record of the row, for the owner that comes last
            float* rcd = p.scratch + ((((size_t)seq * p.nkv + kvh) * p.chunks + chunk) * 16 + row) * (D + 2);
            rcd[c] = o;
            if (c == 0) { rcd[D] = m_all; rcd[D + 1] = l_all; }
          }
        }
        if (chunks_on > 1) {
          // One ticket per (sequence, kv head, owner): the owners of the same rows in the other
          // clusters take theirs when their records are written; the last one adds the records
          // in the order of the chunks.  Nobody waits for anybody.
          volatile int& last_ticket = const_cast<volatile int*>(failed)[1];    // the flag's word neighbour
          __threadfence();
          __syncthreads();
          if (threadIdx.x == 0) {
            int* counter = p.counters + ((size_t)seq * p.nkv + kvh) * 16 + rank;
            const int t = atomicAdd(counter, 1);
            last_ticket = (t == chunks_on - 1) ? 1 : 0;
            if (t == chunks_on - 1) *counter = 0;            // ready for the next launch
          }
          __syncthreads();
          if (last_ticket) {
            __threadfence();
            const float* base_rec = p.scratch + (((size_t)seq * p.nkv + kvh) * p.chunks) * 16 * (D + 2);
            for (int e = threadIdx.x; e < rows_mine * D; e += kThreads) {
              const int c = e % D, row = (e / D) * kSplit + rank;
              float m_all = -INFINITY;
              for (int z = 0; z < chunks_on; ++z) m_all = fmaxf(m_all, __ldcg(base_rec + ((size_t)z * 16 + row) * (D + 2) + D));
              float l_all = 0.f, o = 0.f;
              for (int z = 0; z < chunks_on; ++z) {
                const float* rcd = base_rec + ((size_t)z * 16 + row) * (D + 2);
                const float m = __ldcg(rcd + D);
                const float f = (m == -INFINITY) ? 0.f : exp2f(m - m_all);
                l_all += __ldcg(rcd + D + 1) * f;
                o += __ldcg(rcd + c) * f;
              }
              p.out[(size_t)tok * p.out_stride + (size_t)(kvh * G + row) * D + c] = __float2bfloat16_rn(l_all > 0.f ? o / l_all : 0.f);
            }
          }
        }
      }
      return;
    }
    cluster_sync_all();
    // ---- merge: element e of the group's output from all records, CTA after CTA, warp after warp
    const int live_rows = min(16, G - rb);
    const uint32_t rec_addr = smem_u32(rec);
    const int n_rec = kSplit * kConsumers;
    for (int e = rank * kThreads + threadIdx.x; e < live_rows * D; e += kSplit * kThreads) {
      const int row = e / D, c = e % D;
      auto rec_of = [&](int i) { return rec_addr + (uint32_t)(((i % kConsumers) * 16 + row) * kRec) * 4u; };
      float m_all = -INFINITY;
      for (int i0 = 0; i0 < n_rec; i0 += 8) {                // the records' maxima, eight loads in flight
        float m[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          m[i] = i0 + i < n_rec ? ld_peer_f32(rec_of(i0 + i) + D * 4u, (uint32_t)((i0 + i) / kConsumers)) : -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) m_all = fmaxf(m_all, m[i]);
      }
      float l_all = 0.f, o = 0.f;
      for (int i0 = 0; i0 < n_rec; i0 += 8) {
        float m[8], l[8], v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool on = i0 + i < n_rec;
          const uint32_t a = rec_of(on ? i0 + i : 0), peer = (uint32_t)((on ? i0 + i : 0) / kConsumers);
          m[i] = on ? ld_peer_f32(a + D * 4u, peer) : -INFINITY;
          l[i] = on ? ld_peer_f32(a + (D + 1) * 4u, peer) : 0.f;
          v[i] = on ? ld_peer_f32(a + (uint32_t)c * 4u, peer) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float f = (m[i] == -INFINITY) ? 0.f : exp2f(m[i] - m_all);
          l_all += l[i] * f;
          o += v[i] * f;
        }
      }
      p.out[(size_t)tok * p.out_stride + (size_t)(kvh * G + rb + row) * D + c] = __float2bfloat16_rn(l_all > 0.f ? o / l_all : 0.f);
    }
    cluster_sync_all();                                    // the records stay until every peer has read them
    // the next pass's TMA writes land where ordinary stores and loads have just been
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* ptr; int d, page_size, nkv, num_pages, run;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d == o.d && page_size == o.page_size && nkv == o.nkv && num_pages == o.num_pages && run == o.run;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    for (int v : {k.d, k.page_size, k.nkv, k.num_pages, k.run}) h = h * 1000003u ^ std::hash<int>()(v);
    return h;
  }
};

// The cache as (d, key in page, kv head, page); a box is up to 32 keys of one page and head,
// one slice of the head; `run` pages of fewer keys that follow one another make one box.
int cache_map(CUtensorMap* out, const void* ptr, int d, int page_size, int nkv, int num_pages, int run) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  const MapKey key{ptr, d, page_size, nkv, num_pages, run};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail("attention decode: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)page_size, (cuuint64_t)nkv, (cuuint64_t)num_pages};
  const cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)d * 2 * page_size, (cuuint64_t)d * 2 * page_size * nkv};
  const cuuint32_t box[4] = {64, (cuuint32_t)(page_size < kKeys ? page_size : kKeys), 1, (cuuint32_t)run};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("attention decode: cuTensorMapEncodeTiled failed with code %d", (int)r);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// Ring, alignment slack, barriers and the flag; the records that a cluster sends to this CTA follow.
template <int D, int STAGES>
constexpr size_t ring_bytes() { return (size_t)STAGES * 2 * (D / 64) * kKeys * 128 + 1024 + (2 * STAGES + 2) * 8; }

// Rows of a group of `group` query heads that one CTA of a cluster of `split` owns at most,
// and the bytes of the records sent to it (none when the records stay where they are).
inline int rows_cap_of(int group, int split) { return (split > 1 && group <= 16) ? (group + split - 1) / split : 0; }
inline size_t inbox_bytes(int d, int group, int split) { return (size_t)split * rows_cap_of(group, split) * (d + 4) * 4; }

template <int D, int STAGES>
int configure() {
  static OncePerDevice once;
  if (once.first()) {
    constexpr size_t smem = ring_bytes<D, STAGES>() + (size_t)2 * kMaxSplit * (D + 4) * 4;   // the most a launch asks for
    static_assert(smem <= 227 * 1024, "tile ring does not fit shared memory");
    cudaError_t e = cudaFuncSetAttribute(decode_kernel<D, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) once.forget();
    if (e != cudaSuccess) return fail("attention decode: cannot reserve %zu bytes of shared memory", smem);
    cudaFuncSetAttribute(decode_kernel<D, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(decode_kernel<D, STAGES>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  }
  return 0;
}

// Clusters of `split` CTAs of this kernel, each with `extra` more bytes of shared memory, that
// the device holds at a time (0 if it cannot tell or cannot run them).
template <int D, int STAGES>
int active_clusters(int split, size_t extra) {
  static std::unordered_map<long long, int> cache;
  static std::mutex mu;
  if (split < 1 || split > kMaxSplit) return 0;
  const long long key = (long long)extra * 64 + split;
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (configure<D, STAGES>()) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(split, 64, 8);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = ring_bytes<D, STAGES>() + extra;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, decode_kernel<D, STAGES>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  if (n < 0) n = 0;
  cache.emplace(key, n);
  return n;
}

template <int D, int STAGES>
int launch(const CUtensorMap (&m)[4], const Params& p, size_t extra, cudaStream_t stream) {
  if (configure<D, STAGES>()) return -1;
  ilb::launch_cluster(decode_kernel<D, STAGES>, dim3(p.split, p.nkv, p.n_seqs * p.chunks), dim3(kThreads), ring_bytes<D, STAGES>() + extra, stream,
                      p.split, m[0], m[1], m[2], m[3], p);
  return check_launch("attention decode");
}

// The ways a sequence's tiles are dealt out and the depth of the tile ring: as many CTAs as
// fit the device at once, and the shared memory that this leaves to each of them.
constexpr int kMaxChunks = 8;

// `long_context`: the step's longest sequence is long enough for several clusters per
// (sequence, kv head) to pay; the launch is then shaped for the most CTAs at work, not for the
// widest cluster.
template <int D>
void plan_for(int n_seqs, int nq, int nkv, int long_context, int& split, int& stages, int& chunks) {
  const long long pairs = (long long)n_seqs * nkv;
  const int group = nq / nkv;
  split = kMaxSplit;
  while (split > 1 && active_clusters<D, 3>(split, inbox_bytes(D, group, split)) < pairs) split /= 2;
  chunks = 1;
  if (long_context && split > 1 && group <= 16) {
    long long best = 0;
    int best_split = split;
    for (int s = split; s >= 2; s /= 2) {
      long long c = active_clusters<D, 3>(s, inbox_bytes(D, group, s)) / pairs;
      c = c > kMaxChunks ? kMaxChunks : c;
      if (c * s > best) { best = c * s; best_split = s; chunks = (int)c; }
    }
    split = best_split;
  }
  const size_t extra = inbox_bytes(D, group, split);
  const long long clusters = pairs * chunks;
  stages = active_clusters<D, 12>(split, extra) >= clusters ? 12 : active_clusters<D, 6>(split, extra) >= clusters ? 6 : 3;
}

template <int D>
int launch_for(const CUtensorMap (&m)[4], Params& p, int long_context, long long scratch_floats, long long n_counters, cudaStream_t stream) {
  int stages = 3;
  plan_for<D>(p.n_seqs, p.nq, p.nkv, long_context, p.split, stages, p.chunks);
  const int group = p.nq / p.nkv;
  if (p.chunks > 1) {
    const long long need_f = (long long)p.n_seqs * p.nkv * p.chunks * 16 * (D + 2), need_c = (long long)p.n_seqs * p.nkv * 16;
    if (p.scratch == nullptr || p.counters == nullptr || need_f > scratch_floats || need_c > n_counters)
      plan_for<D>(p.n_seqs, p.nq, p.nkv, 0, p.split, stages, p.chunks);       // no room for the records: one cluster each
  }
  p.rows_cap = rows_cap_of(group, p.split);
  const size_t extra = inbox_bytes(D, group, p.split);
  if (stages == 12) return launch<D, 12>(m, p, extra, stream);
  if (stages == 6) return launch<D, 6>(m, p, extra, stream);
  return launch<D, 3>(m, p, extra, stream);
}

}  // namespace

// Geometry this kernel is built for; everything else takes the ticketed kernel of attention_flash.
ILB_EXPORT int ilb_attention_decode_tma_supported(int nq, int nkv, int d, int page_size) {
  if (nkv <= 0 || nq <= 0 || nq % nkv != 0) return 0;
  return ((d == 64 || d == 128) && (page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128)) ? 1 : 0;
}

// The cluster size and ring depth a launch of this geometry would get (for tests and notes).
ILB_EXPORT int ilb_attention_decode_plan(int n_seqs, int nq, int nkv, int d, int page_size, int long_context, int* split, int* stages,
                                         int* chunks) {
  ILB_REQUIRE(ilb_attention_decode_tma_supported(nq, nkv, d, page_size) && n_seqs > 0 && split && stages && chunks,
              "attention decode: no plan for this geometry");
  if (d == 64) plan_for<64>(n_seqs, nq, nkv, long_context, *split, *stages, *chunks);
  else plan_for<128>(n_seqs, nq, nkv, long_context, *split, *stages, *chunks);
  return 0;
}

// 32-bit elements of scratch and counters that a launch of this geometry can use (it runs
// without them, one cluster per sequence and kv head, when given less).
ILB_EXPORT long long ilb_attention_decode_scratch_floats(int n_seqs, int nkv, int d) {
  return (long long)n_seqs * nkv * kMaxChunks * 16 * (d + 2);
}
ILB_EXPORT long long ilb_attention_decode_counters(int n_seqs, int nkv) { return (long long)n_seqs * nkv * 16; }

namespace {
int decode_common(const void* q, const void* qkv, int qkv_stride, const float* q_weight, const float* k_weight, float eps,
                  const float* rope, int write_kv, void* out, const void* k_cache, const void* v_cache, const int* positions,
                  const int* cu_q, const int* block_table, int max_blocks, int page_size, int num_pages, int window,
                  float scale, int n_seqs, int nq, int nkv, int d, int q_stride, int out_stride, int long_context,
                  float* scratch, long long scratch_floats, int* counters, long long n_counters, int* error_flag, cudaStream_t stream) {
  ILB_REQUIRE(ilb_attention_decode_tma_supported(nq, nkv, d, page_size),
              "attention decode: heads %d/%d, head size %d, page size %d are not built", nq, nkv, d, page_size);
  ILB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && nkv <= 65535 && max_blocks > 0 && num_pages > 0 && window >= 0,
              "attention decode: bad sizes");
  ILB_REQUIRE(((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0), "attention decode: misaligned cache");
  if (qkv != nullptr)
    ILB_REQUIRE(qkv_stride % 2 == 0 && qkv_stride >= (nq + 2 * nkv) * d && ((uintptr_t)qkv % 4 == 0) &&
                ((uintptr_t)rope % 8 == 0) && eps > 0.f, "attention decode: bad fused inputs");
  else
    ILB_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q % 4 == 0), "attention decode: misaligned operands");
  CUtensorMap m[4];                      // K, V, and the same with boxes of two pages
  const int run = page_size < kKeys ? kKeys / page_size : 1;
  if (cache_map(&m[0], k_cache, d, page_size, nkv, num_pages, 1)) return -1;
  if (cache_map(&m[1], v_cache, d, page_size, nkv, num_pages, 1)) return -1;
  if (cache_map(&m[2], k_cache, d, page_size, nkv, num_pages, run)) return -1;
  if (cache_map(&m[3], v_cache, d, page_size, nkv, num_pages, run)) return -1;
  Params p{};
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out;
  p.positions = positions; p.cu_q = cu_q; p.block_table = block_table; p.error_flag = error_flag;
  p.max_blocks = max_blocks; p.n_seqs = n_seqs; p.nq = nq; p.nkv = nkv; p.window = window;
  p.q_stride = q_stride; p.out_stride = out_stride; p.page_size = page_size; p.num_pages = num_pages;
  p.split = 1; p.scale_log2 = scale * kLog2e;
  p.qkv = (const __nv_bfloat16*)qkv; p.qkv_stride = qkv_stride; p.q_weight = q_weight; p.k_weight = k_weight; p.eps = eps;
  p.rope = (const float2*)rope;
  p.k_write = (qkv != nullptr && write_kv) ? (__nv_bfloat16*)const_cast<void*>(k_cache) : nullptr;
  p.v_write = (qkv != nullptr && write_kv) ? (__nv_bfloat16*)const_cast<void*>(v_cache) : nullptr;
  p.chunks = 1; p.scratch = scratch; p.counters = counters;
  return d == 64 ? launch_for<64>(m, p, long_context, scratch_floats, n_counters, stream)
                 : launch_for<128>(m, p, long_context, scratch_floats, n_counters, stream);
}
}  // namespace

ILB_EXPORT int ilb_attention_decode_tma(const void* q, void* out, const void* k_cache, const void* v_cache,
                                        const int* positions, const int* cu_q, const int* block_table,
                                        int max_blocks, int page_size, int num_pages, int window, float scale,
                                        int n_seqs, int nq, int nkv, int d, int q_stride, int out_stride,
                                        int long_context, float* scratch, long long scratch_floats, int* counters, long long n_counters,
                                        int* error_flag, cudaStream_t stream) {
  return decode_common(q, nullptr, 0, nullptr, nullptr, 1.f, nullptr, 0, out, k_cache, v_cache, positions, cu_q, block_table,
                       max_blocks, page_size, num_pages, window, scale, n_seqs, nq, nkv, d, q_stride, out_stride, long_context,
                       scratch, scratch_floats, counters, n_counters, error_flag, stream);
}

// The same with the step's q/k/v taken from the fused projection output `qkv`
// [tokens, (nq + 2 nkv) d]: per-head RMSNorm (q_weight / k_weight [d], or null), rotation over
// the whole head (rope [tokens, d/2, 2] cos/sin, or null), and, if write_kv, the new key and
// value stored to the cache.  What qk_norm_rope.cu and this kernel do in two launches.
ILB_EXPORT int ilb_attention_decode_fused(const void* qkv, int qkv_stride, const float* q_weight, const float* k_weight,
                                          float eps, const float* rope, int write_kv, void* out, void* k_cache,
                                          void* v_cache, const int* positions, const int* cu_q, const int* block_table,
                                          int max_blocks, int page_size, int num_pages, int window, float scale,
                                          int n_seqs, int nq, int nkv, int d, int out_stride, int long_context,
                                          float* scratch, long long scratch_floats, int* counters, long long n_counters, int* error_flag,
                                          cudaStream_t stream) {
  ILB_REQUIRE(qkv != nullptr, "attention decode: no projection output");
  return decode_common(nullptr, qkv, qkv_stride, q_weight, k_weight, eps, rope, write_kv, out, k_cache, v_cache, positions,
                       cu_q, block_table, max_blocks, page_size, num_pages, window, scale, n_seqs, nq, nkv, d, 0, out_stride,
                       long_context, scratch, scratch_floats, counters, n_counters, error_flag, stream);
}

ILB_DEFINE_LAST_ERROR()
