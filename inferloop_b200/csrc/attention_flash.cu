// Causal grouped-query attention over the paged bfloat16 cache on tensor cores
// (mma.sync m16n8k16, 32-bit accumulation and softmax), for prefill and for decode.
//
// Rows of a tile are (token, query head within its kv group) pairs of ONE kv head, so the
// keys and values of that head are loaded once for the whole group.  Keys and values come
// from the cache pages through the block table into shared memory with cp.async, 64 keys a
// tile; S = Q K^T and O += P V run as m16n8k16 MMAs with the online-softmax rescaling in
// between, all statistics in 32-bit, exponentials as exp2 of log2(e)-scaled scores.
//
//   prefill  one CTA = 64 rows (4 warps x 16) of one sequence and kv head; it walks the
//            key tiles from the window start to the last row's position (double buffered).
//   decode   one token per sequence: the keys are cut into chunks of `chunk` keys whose
//            boundaries depend on the key index alone; one CTA per (kv head, sequence,
//            chunk) walks its chunk in 64-key tiles (double buffered), each of its 4 warps
//            taking 16 keys of every tile.  A CTA parks (max, sum, O) of its chunk
//            in a 32-bit scratch buffer and takes a ticket; the CTA with the last ticket of
//            a (sequence, kv head) merges the chunks in chunk order and writes the output.
//            Nothing ever waits on another CTA.
//
// The reference's counterparts: `attention::decode_tiled` (prefill, query tiles on MMAs),
// `partial_gqa_lanes` + `merge_gqa` (split-KV decode with the group's heads padded to 16
// MMA rows) in crates/backend/cuda-kernels/src/tile/attention/
// resident_attention_prefill_kernels.rs:378-469 and resident_attention_decode_kernels.rs:
// 131-226, :417-451, :497-598; masked scores are dropped and rows without keys give 0
// (:460-468 of the former).  Formula: crates/testing/cpu/reference-ops/src/kernels.rs:251-297.
#include <math.h>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

namespace {

constexpr int kTileKeys = 64;
constexpr int kWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct Cache {
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int page_size, num_pages, nkv;
};

// Copy keys [key0, key0 + 64) of kv head `kvh` of BOTH caches into two [64][D + 8] tiles;
// rows whose key is outside [lo, hi) or whose page is not held are zero-filled.  NT
// threads take part; each owns one 16-byte column of the rows it copies, so its page
// lookups are independent of one another and are issued together.
template <int D, int NT>
__device__ __forceinline__ void load_tiles(__nv_bfloat16* kdst, __nv_bfloat16* vdst, const Cache& c,
                                           const int* __restrict__ table, int max_blocks, int kvh, int key0,
                                           int lo, int hi, int tid) {
  constexpr int kStride = D + 8;
  constexpr int kChunks = D / 8;                 // 16-byte pieces per row
  if constexpr (NT % kChunks == 0 && (kTileKeys * kChunks) % NT == 0) {
    constexpr int kRowsPerIter = NT / kChunks;
    constexpr int kIters = kTileKeys / kRowsPerIter;
    const int ch = tid % kChunks, r0 = tid / kChunks;
    size_t off[kIters];
    int bytes[kIters];
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int key = key0 + r0 + it * kRowsPerIter;
      const int blk = key / c.page_size;
      const bool in = key >= lo && key < hi && blk < max_blocks;
      const int page = in ? __ldg(table + blk) : -1;
      const bool ok = page >= 0 && page < c.num_pages;
      off[it] = ok ? (((size_t)page * c.nkv + kvh) * c.page_size + (key % c.page_size)) * D + ch * 8 : 0;
      bytes[it] = ok ? 16 : 0;
    }
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int r = r0 + it * kRowsPerIter;
      cp_async_16(smem_u32(kdst + r * kStride + ch * 8), c.k + off[it], bytes[it]);
      cp_async_16(smem_u32(vdst + r * kStride + ch * 8), c.v + off[it], bytes[it]);
    }
  } else {
    for (int idx = tid; idx < kTileKeys * kChunks; idx += NT) {
      const int r = idx / kChunks, ch = idx % kChunks;
      const int key = key0 + r;
      size_t off = 0;
      int bytes = 0;
      if (key >= lo && key < hi) {
        const int blk = key / c.page_size;
        const int page = blk < max_blocks ? __ldg(table + blk) : -1;
        if (page >= 0 && page < c.num_pages) {
          off = (((size_t)page * c.nkv + kvh) * c.page_size + (key % c.page_size)) * D + ch * 8;
          bytes = 16;
        }
      }
      cp_async_16(smem_u32(kdst + r * kStride + ch * 8), c.k + off, bytes);
      cp_async_16(smem_u32(vdst + r * kStride + ch * 8), c.v + off, bytes);
    }
  }
}

// State of 16 rows held by one warp: thread (g = lane / 4, t = lane % 4) owns rows g and
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

// NB * 8 keys (rows of `ks` / `vs`, the first being key `key0`) for one warp's 16 rows.
// pos[2] / lo[2]: last and first visible key of rows g and g + 8 (pos < lo hides
// everything).  `hi`: keys >= hi do not exist.
template <int D, int NB>
__device__ __forceinline__ void tile_step(RowState<D>& st, const uint32_t (&q)[D / 16][4],
                                          const __nv_bfloat16* ks, const __nv_bfloat16* vs, int key0,
                                          const int (&pos)[2], const int (&lo)[2], int hi, float scale_log2, int lane) {
  static_assert(NB % 2 == 0, "keys are consumed 16 at a time");
  constexpr int kStride = D + 8;
  const int t = lane & 3;
  float s[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nb][e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D / 16; kk += 2) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4(smem_u32(ks + (nb * 8 + (lane & 7)) * kStride + kk * 16 + (lane >> 3) * 8), r0, r1, r2, r3);
      mma_16816(s[nb], q[kk], r0, r1);
      mma_16816(s[nb], q[kk + 1], r2, r3);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + nb * 8 + 2 * t + (e & 1);
      const int r = e >> 1;
      const bool ok = key <= pos[r] && key >= lo[r] && key < hi;
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
  for (int nb = 0; nb < NB; ++nb)
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
#pragma unroll
  for (int kb = 0; kb < NB / 2; ++kb) {            // 16 keys per step
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
    a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
    a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
    a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
    for (int nd = 0; nd < D / 16; ++nd) {
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4_trans(smem_u32(vs + (kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kStride + nd * 16 + (lane >> 4) * 8),
                        r0, r1, r2, r3);
      mma_16816(st.o[2 * nd], a, r0, r1);
      mma_16816(st.o[2 * nd + 1], a, r2, r3);
    }
  }
}

// Q rows g and g + 8 of a warp as A fragments; a null pointer gives a zero row.
template <int D>
__device__ __forceinline__ void load_q(uint32_t (&q)[D / 16][4], const __nv_bfloat16* row0, const __nv_bfloat16* row1, int lane) {
  const int t = lane & 3;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int c = kk * 16 + 2 * t;
    q[kk][0] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c) : 0u;
    q[kk][1] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c) : 0u;
    q[kk][2] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c + 8) : 0u;
    q[kk][3] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c + 8) : 0u;
  }
}

// ------------------------------------------------------------------ prefill
struct PrefillParams {
  const __nv_bfloat16* q; __nv_bfloat16* out;
  Cache cache;
  const int* positions; const int* cu_q; const int* block_table;
  int max_blocks, n_seqs, nq, window, q_stride, out_stride;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kWarps * 32)
prefill_kernel(const PrefillParams p) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  constexpr int kStride = D + 8;
  constexpr int kTileElems = kTileKeys * kStride;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [2][K, V][64][D + 8]
  const int G = p.nq / p.cache.nkv;
  const int kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

  // which sequence and which 64-row tile of it; the last tiles of a prompt see the most
  // keys, so they are handed out first and the short ones fill the tail of the launch
  int seq = 0, tile = (int)gridDim.x - 1 - (int)blockIdx.x;
  for (; seq < p.n_seqs; ++seq) {
    const int rows = (p.cu_q[seq + 1] - p.cu_q[seq]) * G;
    const int tiles = (rows + 63) / 64;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (seq >= p.n_seqs) return;
  const int tok0 = p.cu_q[seq], q_len = p.cu_q[seq + 1] - tok0;
  const int* table = p.block_table + (size_t)seq * p.max_blocks;

  // this thread's two rows
  int pos[2], lo[2], tok[2], head[2];
  bool live[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = tile * 64 + warp * 16 + g + 8 * r;
    const int tl = row / G;
    live[r] = tl < q_len;
    tok[r] = tok0 + (live[r] ? tl : 0);
    head[r] = kvh * G + row % G;
    pos[r] = live[r] ? p.positions[tok[r]] : -1;
    lo[r] = (live[r] && p.window > 0 && pos[r] + 1 > p.window) ? pos[r] + 1 - p.window : 0;
    if (!live[r]) lo[r] = 0;
  }
  // keys the whole CTA needs: from the smallest window start to the largest position
  const int first_tl = (tile * 64) / G;
  const int last_tl = min(q_len - 1, (tile * 64 + 63) / G);
  const int pos_first = p.positions[tok0 + first_tl], pos_last = p.positions[tok0 + last_tl];
  const int key_lo = (p.window > 0 && pos_first + 1 > p.window) ? pos_first + 1 - p.window : 0;
  const int hi = pos_last + 1;

  uint32_t q[D / 16][4];
  load_q<D>(q, live[0] ? p.q + (size_t)tok[0] * p.q_stride + (size_t)head[0] * D : nullptr,
            live[1] ? p.q + (size_t)tok[1] * p.q_stride + (size_t)head[1] * D : nullptr, lane);
  RowState<D> st;
  st.init();

  const int first_tile = key_lo / kTileKeys, n_tiles = (hi + kTileKeys - 1) / kTileKeys - first_tile;
  auto issue = [&](int i) {
    __nv_bfloat16* buf = smem + (i & 1) * 2 * kTileElems;
    const int key0 = (first_tile + i) * kTileKeys;
    load_tiles<D, kWarps * 32>(buf, buf + kTileElems, p.cache, table, p.max_blocks, kvh, key0, key_lo, hi, threadIdx.x);
    cp_async_commit();
  };
  issue(0);
  for (int i = 0; i < n_tiles; ++i) {
    if (i + 1 < n_tiles) { issue(i + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const __nv_bfloat16* buf = smem + (i & 1) * 2 * kTileElems;
    const int key0 = (first_tile + i) * kTileKeys;
    // a warp whose rows cannot see this tile skips the math (the barrier is kept)
    const int wpos = __reduce_max_sync(0xffffffffu, max(pos[0], pos[1]));
    if (key0 <= wpos) tile_step<D, 8>(st, q, buf, buf + kTileElems, key0, pos, lo, hi, p.scale_log2, lane);
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = st.l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (!live[r]) continue;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = p.out + (size_t)tok[r] * p.out_stride + (size_t)head[r] * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16(st.o[i][2 * r] * inv, st.o[i][2 * r + 1] * inv);
  }
}

// ------------------------------------------------------------------ decode
struct DecodeParams {
  const __nv_bfloat16* q; __nv_bfloat16* out;
  Cache cache;
  const int* positions; const int* cu_q; const int* block_table;
  float* scratch;      // [seqs][nkv][chunks][G][D + 2]
  int* tickets;        // [seqs * nkv], zero between launches
  int max_blocks, n_seqs, nq, window, q_stride, out_stride, chunk, max_chunks, rows16;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kWarps * 32)
decode_kernel(const DecodeParams p) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  constexpr int kStride = D + 8;
  constexpr int kTileElems = kTileKeys * kStride;
  constexpr int kRec = D + 2;                      // O row, then max and sum
  constexpr int kKeysPerWarp = kTileKeys / kWarps; // each warp takes 16 keys of every tile
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [2][K, V][64][D + 8]
  float* merge = reinterpret_cast<float*>(smem_raw);                  // reused once the tiles are consumed
  __shared__ int s_last;
  const int G = p.nq / p.cache.nkv;
  const int kvh = blockIdx.x, seq = blockIdx.y, chunk_i = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tok = p.cu_q[seq];
  if (p.cu_q[seq + 1] - tok != 1) return;          // decode handles one token per sequence
  const int pos = p.positions[tok];
  const int lo = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
  const int hi = pos + 1;
  const int c_lo = lo / p.chunk, c_hi = pos / p.chunk;
  if (chunk_i < c_lo || chunk_i > c_hi) return;
  const int n_chunks = c_hi - c_lo + 1;
  const int* table = p.block_table + (size_t)seq * p.max_blocks;
  const int key_begin = chunk_i * p.chunk;
  const int key_end = min(key_begin + p.chunk, hi);
  const int n_tiles = (key_end - key_begin + kTileKeys - 1) / kTileKeys;
  float* rec_base = p.scratch + (((size_t)seq * p.cache.nkv + kvh) * p.max_chunks) * (size_t)(G * kRec);

  auto issue = [&](int i) {
    __nv_bfloat16* buf = smem + (i & 1) * 2 * kTileElems;
    const int key0 = key_begin + i * kTileKeys;
    load_tiles<D, kWarps * 32>(buf, buf + kTileElems, p.cache, table, p.max_blocks, kvh, key0, lo, key_end, threadIdx.x);
    cp_async_commit();
  };

  for (int rb = 0; rb < p.rows16; rb += 16) {      // 16 query heads of the group at a time
    issue(0);
    if (n_tiles > 1) issue(1);
    RowState<D> st;
    st.init();
    int rpos[2], rlo[2];
    const __nv_bfloat16* qrow[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int h = rb + g + 8 * r;
      const bool live = h < G;
      rpos[r] = live ? pos : -1;
      rlo[r] = lo;
      qrow[r] = live ? p.q + (size_t)tok * p.q_stride + (size_t)(kvh * G + h) * D : nullptr;
    }
    uint32_t q[D / 16][4];
    load_q<D>(q, qrow[0], qrow[1], lane);
    for (int i = 0; i < n_tiles; ++i) {
      if (i + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncthreads();
      const __nv_bfloat16* buf = smem + (i & 1) * 2 * kTileElems;
      const int key0 = key_begin + i * kTileKeys + warp * kKeysPerWarp;
      if (key0 < key_end)
        tile_step<D, kKeysPerWarp / 8>(st, q, buf + warp * kKeysPerWarp * kStride,
                                       buf + kTileElems + warp * kKeysPerWarp * kStride, key0, rpos, rlo, key_end,
                                       p.scale_log2, lane);
      __syncthreads();
      if (i + 2 < n_tiles) issue(i + 2);
    }
    // ---- merge the four warps (fixed order) into the chunk's record
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = st.l[r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      float* row = merge + ((size_t)warp * 16 + g + 8 * r) * kRec;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { row[i * 8 + 2 * t] = st.o[i][2 * r]; row[i * 8 + 2 * t + 1] = st.o[i][2 * r + 1]; }
      if (t == 0) { row[D] = st.m[r]; row[D + 1] = l; }
    }
    __syncthreads();
    float* rec = rec_base + ((size_t)chunk_i * G + rb) * kRec;
    const int live_rows = min(16, G - rb);
    for (int idx = threadIdx.x; idx < live_rows * kRec; idx += kWarps * 32) {
      const int row = idx / kRec, c = idx % kRec;
      float mw[kWarps], m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) { mw[w] = merge[((size_t)w * 16 + row) * kRec + D]; m_all = fmaxf(m_all, mw[w]); }
      float acc = 0.f;
      if (c == D) acc = m_all;
      else {
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float f = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - m_all);
          acc += merge[((size_t)w * 16 + row) * kRec + c] * f;      // c == D + 1 sums l the same way
        }
      }
      rec[idx] = acc;
    }
    __syncthreads();
  }
  if (n_chunks == 1) {
    // the only chunk: its record is the answer (read back through L2 by the writers' block)
    __threadfence_block();
    for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
      const int h = idx / D, c = idx % D;
      const float* rec = rec_base + ((size_t)chunk_i * G + h) * kRec;
      const float l = rec[D + 1];
      p.out[(size_t)tok * p.out_stride + (size_t)(kvh * G + h) * D + c] = __float2bfloat16_rn(l > 0.f ? rec[c] / l : 0.f);
    }
    return;
  }
  // ---- ticket: the last chunk of this (sequence, kv head) merges all chunks in order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* ticket = p.tickets + seq * p.cache.nkv + kvh;
    const int tk = atomicAdd(ticket, 1);
    s_last = (tk == n_chunks - 1) ? 1 : 0;
    if (tk == n_chunks - 1) *ticket = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // weights of the chunks per head: f[h][ci] = 2^(m_ci - M) / L.  One warp per head, one
  // lane per chunk (32 chunks a round), so every record is fetched once and all fetches
  // of a round are in flight together; sums run in chunk order within a lane's stride and
  // are combined by a fixed shuffle tree.
  float* fw = merge;                               // [G][n_chunks]
  for (int h = warp; h < G; h += kWarps) {
    float m_all = -INFINITY;
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
      const int ci = c0 + lane;
      const float mc = ci < n_chunks ? __ldcg(rec_base + ((size_t)(c_lo + ci) * G + h) * kRec + D) : -INFINITY;
      m_all = fmaxf(m_all, mc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
    float l_all = 0.f;
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
      const int ci = c0 + lane;
      float f = 0.f, l = 0.f;
      if (ci < n_chunks) {
        const float* rec = rec_base + ((size_t)(c_lo + ci) * G + h) * kRec;
        const float mc = __ldcg(rec + D);
        l = __ldcg(rec + D + 1);
        f = (mc == -INFINITY) ? 0.f : exp2f(mc - m_all);
        fw[h * n_chunks + ci] = f;
      }
      l_all += l * f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, o);
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    __syncwarp();
    for (int ci = lane; ci < n_chunks; ci += 32) fw[h * n_chunks + ci] *= inv;
  }
  __syncthreads();
  // every output element: its chunks' values, eight fetches in flight per element and the
  // elements of a thread unrolled so that their fetches overlap too
  constexpr int kPerThread = 4;
  for (int base = 0; base < G * D; base += kWarps * 32 * kPerThread) {
    float o[kPerThread];
#pragma unroll
    for (int e = 0; e < kPerThread; ++e) o[e] = 0.f;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {
      float v[kPerThread][8];
#pragma unroll
      for (int e = 0; e < kPerThread; ++e) {
        const int idx = base + e * kWarps * 32 + threadIdx.x;
        const int h = idx / D, c = idx % D;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[e][j] = (idx < G * D && c0 + j < n_chunks) ? __ldcg(rec_base + ((size_t)(c_lo + c0 + j) * G + h) * kRec + c) : 0.f;
      }
#pragma unroll
      for (int e = 0; e < kPerThread; ++e) {
        const int idx = base + e * kWarps * 32 + threadIdx.x;
        const int h = idx < G * D ? idx / D : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) if (c0 + j < n_chunks) o[e] += v[e][j] * fw[h * n_chunks + c0 + j];
      }
    }
#pragma unroll
    for (int e = 0; e < kPerThread; ++e) {
      const int idx = base + e * kWarps * 32 + threadIdx.x;
      if (idx < G * D) {
        const int h = idx / D, c = idx % D;
        p.out[(size_t)tok * p.out_stride + (size_t)(kvh * G + h) * D + c] = __float2bfloat16_rn(o[e]);
      }
    }
  }
}

template <int D> size_t prefill_smem() { return (size_t)2 * 2 * kTileKeys * (D + 8) * 2; }
template <int D> size_t decode_smem() {
  const size_t tiles = (size_t)2 * 2 * kTileKeys * (D + 8) * 2, merge = (size_t)kWarps * 16 * (D + 2) * 4;
  return tiles > merge ? tiles : merge;
}

template <int D>
int launch_prefill(const PrefillParams& p, int n_tiles, cudaStream_t stream) {
  static OncePerDevice once;
  const size_t smem = prefill_smem<D>();
  if (once.first()) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) once.forget();
    if (e != cudaSuccess) return fail("attention prefill: cannot reserve %zu bytes of shared memory", smem);
  }
  ilb::launch(prefill_kernel<D>, dim3(n_tiles, p.cache.nkv), dim3(kWarps * 32), smem, stream, p);
  return check_launch("attention prefill");
}

template <int D>
int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  static OncePerDevice once;
  const size_t smem = decode_smem<D>();
  if (once.first()) {
    cudaError_t e = cudaFuncSetAttribute(decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) once.forget();
    if (e != cudaSuccess) return fail("attention decode: cannot reserve %zu bytes of shared memory", smem);
  }
  ilb::launch(decode_kernel<D>, dim3(p.cache.nkv, p.n_seqs, p.max_chunks), dim3(kWarps * 32), smem, stream, p);
  return check_launch("attention decode");
}

}  // namespace

// Head sizes the tensor-core kernels are built for; any other size takes the exact kernel.
ILB_EXPORT int ilb_attention_flash_supported(int d) { return (d == 32 || d == 64 || d == 96 || d == 128) ? 1 : 0; }

ILB_EXPORT int ilb_attention_prefill(const void* q, void* out, const void* k_cache, const void* v_cache,
                                     const int* positions, const int* cu_q, const int* block_table,
                                     int max_blocks, int page_size, int num_pages, int window, float scale,
                                     int n_seqs, int n_tiles, int nq, int nkv, int d, int q_stride, int out_stride,
                                     cudaStream_t stream) {
  ILB_REQUIRE(ilb_attention_flash_supported(d), "attention prefill: head size %d is not built (32, 64, 96, 128 are)", d);
  ILB_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention prefill: %d query heads are not a multiple of %d kv heads", nq, nkv);
  ILB_REQUIRE(n_seqs > 0 && n_tiles > 0 && nkv <= 65535, "attention prefill: bad grid");
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0, "attention prefill: bad cache geometry");
  ILB_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && ((uintptr_t)q % 4 == 0) && ((uintptr_t)out % 4 == 0) &&
              ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0), "attention prefill: misaligned operands");
  PrefillParams p{(const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                  Cache{(const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, page_size, num_pages, nkv},
                  positions, cu_q, block_table, max_blocks, n_seqs, nq, window, q_stride, out_stride, scale * kLog2e};
  switch (d) {
    case 32: return launch_prefill<32>(p, n_tiles, stream);
    case 64: return launch_prefill<64>(p, n_tiles, stream);
    case 96: return launch_prefill<96>(p, n_tiles, stream);
    default: return launch_prefill<128>(p, n_tiles, stream);
  }
}

// scratch: n_seqs * nkv * max_chunks * (nq / nkv) * (d + 2) floats; tickets: n_seqs * nkv ints, zero.
ILB_EXPORT int ilb_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                    const int* positions, const int* cu_q, const int* block_table,
                                    int max_blocks, int page_size, int num_pages, int window, float scale,
                                    int n_seqs, int nq, int nkv, int d, int q_stride, int out_stride,
                                    int chunk, int max_chunks, float* scratch, long long scratch_floats,
                                    int* tickets, int n_tickets, cudaStream_t stream) {
  ILB_REQUIRE(ilb_attention_flash_supported(d), "attention decode: head size %d is not built (32, 64, 96, 128 are)", d);
  ILB_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention decode: %d query heads are not a multiple of %d kv heads", nq, nkv);
  ILB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && max_chunks > 0 && max_chunks <= 65535, "attention decode: bad grid");
  ILB_REQUIRE(chunk > 0 && chunk % (kWarps * kTileKeys) == 0, "attention decode: chunk %d must be a multiple of %d", chunk, kWarps * kTileKeys);
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0 && window >= 0, "attention decode: bad cache geometry");
  const int G = nq / nkv, rows16 = (G + 15) / 16 * 16;
  ILB_REQUIRE((long long)n_seqs * nkv * max_chunks * G * (d + 2) <= scratch_floats, "attention decode: scratch too small");
  // Every key the block tables can name must fall into one of the chunks: a sequence longer
  // than max_chunks * chunk would wait for chunks that the grid does not hold, and its row
  // would never be written.
  ILB_REQUIRE((long long)max_chunks * chunk >= (long long)max_blocks * page_size,
              "attention decode: %d chunks of %d keys do not cover the %d x %d keys the block tables can name",
              max_chunks, chunk, max_blocks, page_size);
  // The last chunk's merge keeps one weight per (head of the group, chunk) in the shared
  // memory the tiles used.
  const size_t smem_bytes = d == 32 ? decode_smem<32>() : d == 64 ? decode_smem<64>() : d == 96 ? decode_smem<96>() : decode_smem<128>();
  ILB_REQUIRE((long long)G * max_chunks * 4 <= (long long)smem_bytes,
              "attention decode: %d heads a group x %d chunks need %lld bytes of merge weights, the kernel has %zu; "
              "use longer chunks", G, max_chunks, (long long)G * max_chunks * 4, smem_bytes);
  ILB_REQUIRE(n_seqs * nkv <= n_tickets, "attention decode: too few tickets");
  DecodeParams p{(const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                 Cache{(const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, page_size, num_pages, nkv},
                 positions, cu_q, block_table, scratch, tickets, max_blocks, n_seqs, nq, window, q_stride, out_stride,
                 chunk, max_chunks, rows16, scale * kLog2e};
  switch (d) {
    case 32: return launch_decode<32>(p, stream);
    case 64: return launch_decode<64>(p, stream);
    case 96: return launch_decode<96>(p, stream);
    default: return launch_decode<128>(p, stream);
  }
}

// ------------------------------------------------------------------ decode without allocation
// See attention_decode_static.h for who needs this and what it costs.
#include "attention_decode_static.h"
#include <mutex>

// Counters first (they are cleared before every launch), then the chunk records.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_ptr[kMaxDevices] = {};
std::mutex g_static_mu;

// Device address of g_static_scratch on the current device.  In host code the array's name
// is only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
int static_scratch(void** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail("attention decode (static): cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail("attention decode (static): device ordinal %d is outside 0..%d", dev, kMaxDevices - 1);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail("attention decode (static): cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    g_static_ptr[dev] = p;
  }
  *ptr = g_static_ptr[dev];
  return 0;
}
}  // namespace

ILB_EXPORT int ilb_attention_decode_static(const void* q, void* out, const void* k_cache, const void* v_cache,
                                           const int* positions, const int* cu_q, const int* block_table,
                                           int max_blocks, int page_size, int num_pages, int window, float scale,
                                           int n_seqs, int nq, int nkv, int d, int q_stride, int out_stride,
                                           int chunk, int max_chunks, cudaStream_t stream) {
  ILB_REQUIRE(n_seqs > 0 && nq > 0 && nkv > 0 && nq % nkv == 0 && d > 0 && max_chunks > 0,
              "attention decode (static): bad sizes");
  const long long need = (long long)n_seqs * nkv * max_chunks * (nq / nkv) * (d + 2);
  ILB_REQUIRE(need <= (long long)kStaticScratchFloats,
              "attention decode (static): %d sequences x %d kv heads x %d chunks x %d heads x (%d + 2) = %lld floats of "
              "scratch exceed the built-in %d; use ilb_attention_decode with a buffer of your own",
              n_seqs, nkv, max_chunks, nq / nkv, d, need, (int)kStaticScratchFloats);
  ILB_REQUIRE((long long)n_seqs * nkv <= (long long)kStaticTickets,
              "attention decode (static): %d sequences x %d kv heads exceed the built-in %d counters",
              n_seqs, nkv, (int)kStaticTickets);
  void* base = nullptr;
  if (static_scratch(&base)) return -1;
  int* tickets = reinterpret_cast<int*>(base);
  float* records = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + (size_t)kStaticTickets * 4);
  // The counters must read zero when the kernel starts, whatever an earlier call left.
  cudaError_t e = cudaMemsetAsync(tickets, 0, (size_t)kStaticTickets * 4, stream);
  if (e != cudaSuccess) return fail("attention decode (static): clearing the counters failed: %s", cudaGetErrorString(e));
  return ilb_attention_decode(q, out, k_cache, v_cache, positions, cu_q, block_table, max_blocks, page_size, num_pages,
                              window, scale, n_seqs, nq, nkv, d, q_stride, out_stride, chunk, max_chunks, records,
                              (long long)kStaticScratchFloats, tickets, (int)kStaticTickets, stream);
}

ILB_DEFINE_LAST_ERROR()
