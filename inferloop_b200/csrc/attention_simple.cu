// Causal grouped-query attention over the paged cache, any batch shape, exact 32-bit.
//
// One block per (token, query head).  The token at position p of sequence s reads the keys
// of positions lo..p of that sequence from the cache (this step's own keys are already
// there), lo = max(0, p - window + 1) with a window, else 0.  Scores, the running maximum,
// exponentials, sums and the weighted value sum are all 32-bit; the split of the keys over
// the block's warps depends on lo and p alone, so the result at a position never depends
// on what else is in the batch or on how the tokens were cut into steps.
//
// Reference formula: s_j = q.k_j / sqrt(d), p = softmax(s), o = sum p_j v_j, query head h
// uses kv head h / (nq / nkv); window start (p + 1).saturating_sub(w)
// (crates/testing/cpu/reference-ops/src/kernels.rs:251-297).
#include <math.h>
#include "common.cuh"

using namespace ilb;

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_simple_kernel(const TQ* __restrict__ q, TQ* __restrict__ out,
                              const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                              const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                              const int* __restrict__ block_table, int max_blocks, int page_size,
                              int num_pages, int window, float scale, int nq, int nkv, int d,
                              int q_stride, int out_stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float qs[kMaxHeadDim];
  __shared__ float red_m[kWarps], red_l[kWarps];
  __shared__ float red_acc[kWarps][kMaxHeadDim];
  const int t = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h / (nq / nkv);
  const int p = positions[t];
  const int seq = seq_of_token[t];
  const int lo = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
  const int* table = block_table + (size_t)seq * max_blocks;

  for (int i = threadIdx.x; i < d; i += blockDim.x)
    qs[i] = to_float(q[(size_t)t * q_stride + (size_t)h * d + i]);
  __syncthreads();

  constexpr int R = kMaxHeadDim / 32;
  float acc[R];
#pragma unroll
  for (int i = 0; i < R; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int n_keys = p - lo + 1;
  const int n_tiles = (n_keys + 31) / 32;
  for (int tile = warp; tile < n_tiles; tile += kWarps) {
    const int j = lo + tile * 32 + lane;
    const bool valid = j <= p;
    float s = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      if (page >= 0 && page < num_pages) {
        const TC* kr = k_cache + (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * d;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_float(kr[i]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < R; ++i) acc[i] *= corr;
    m = m_new;
    const int count = min(32, p - (lo + tile * 32) + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float w = __shfl_sync(0xffffffffu, pj, jj);
      const int key = lo + tile * 32 + jj;
      const int page = table[key / page_size];
      if (page < 0 || page >= num_pages) continue;
      const TC* vr = v_cache + (((size_t)page * nkv + kvh) * page_size + (key % page_size)) * d;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int c = lane + 32 * i;
        if (c < d) acc[i] = fmaf(w, to_float(vr[c]), acc[i]);
      }
    }
  }
  if (lane == 0) { red_m[warp] = m; red_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int c = lane + 32 * i;
    if (c < d) red_acc[warp][c] = acc[i];
  }
  __syncthreads();
  float m_all = -INFINITY;
  for (int w = 0; w < kWarps; ++w) m_all = fmaxf(m_all, red_m[w]);
  float f[kWarps], l_all = 0.f;
  for (int w = 0; w < kWarps; ++w) {
    f[w] = (red_m[w] == -INFINITY) ? 0.f : expf(red_m[w] - m_all);
    l_all += red_l[w] * f[w];
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float o = 0.f;
    for (int w = 0; w < kWarps; ++w) o += red_acc[w][c] * f[w];
    // A row whose keys are all unreachable gives 0, as the reference does
    // (crates/backend/cuda-kernels/src/tile/attention/resident_attention_prefill_kernels.rs:460-468).
    out[(size_t)t * out_stride + (size_t)h * d + c] = from_float<TQ>(l_all > 0.f ? o / l_all : 0.f);
  }
}

ILB_EXPORT int ilb_paged_attention_simple(
    const void* q, void* out, int dtype, const void* k_cache, const void* v_cache, int cache_dtype,
    const int* positions, const int* seq_of_token, const int* block_table, int max_blocks,
    int page_size, int num_pages, int window, float scale, int n_tokens, int nq, int nkv, int d,
    int q_stride, int out_stride, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0, "attention: bad sizes");
  ILB_REQUIRE(nq % nkv == 0, "attention: %d query heads are not a multiple of %d kv heads", nq, nkv);
  ILB_REQUIRE(d <= kMaxHeadDim, "attention: head size %d exceeds %d", d, kMaxHeadDim);
  ILB_REQUIRE(nq <= 65535, "attention: too many heads");
  ILB_REQUIRE(page_size > 0 && max_blocks > 0 && num_pages > 0, "attention: bad cache geometry");
  ILB_REQUIRE(window >= 0, "attention: negative window");
  ILB_REQUIRE(q_stride >= nq * d && out_stride >= nq * d, "attention: strides too small");
  if (n_tokens == 0) return 0;
  dim3 grid(n_tokens, nq);
#define ILB_LAUNCH(TQ, TC)                                                                    \
  ilb::launch(paged_attention_simple_kernel<TQ, TC>, dim3(grid), dim3(kWarps * 32), 0, stream,                      \
      (const TQ*)q, (TQ*)out, (const TC*)k_cache, (const TC*)v_cache, positions, seq_of_token, \
      block_table, max_blocks, page_size, num_pages, window, scale, nq, nkv, d, q_stride,      \
      out_stride)
  if (dtype == kF32 && cache_dtype == kF32) ILB_LAUNCH(float, float);
  else if (dtype == kBF16 && cache_dtype == kBF16) ILB_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == kF32 && cache_dtype == kBF16) ILB_LAUNCH(float, __nv_bfloat16);
  else if (dtype == kBF16 && cache_dtype == kF32) ILB_LAUNCH(__nv_bfloat16, float);
  else return fail("attention: unsupported dtypes %d/%d", dtype, cache_dtype);
#undef ILB_LAUNCH
  return check_launch("paged_attention_simple");
}

ILB_DEFINE_LAST_ERROR()
