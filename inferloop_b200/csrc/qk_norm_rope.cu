// Fused per-head q/k RMSNorm + rotary position encoding + paged KV-cache write.
//
// Input is the fused projection output qkv[T, (nq + 2*nkv) * d].  For every token and
// head this kernel, in 32-bit:
//   q, k heads: optional RMSNorm over the head (weight [d] shared by all heads), then the
//               half-split rotation of the first `rotary_dim` elements;
//   q -> q_out[T, nq*d];  k, v -> the cache page of the token's position.
// The reference runs these as three launches (norm_rows, prefill_rope, attention::append;
// crates/backend/cuda-kernels/src/tile/state/aux_kernels.rs:104-200 and
// tile/attention/resident_attention_prefill_kernels.rs:170-245).  Formulas: per-head norm
// before the rotation (crates/model/recipes/src/decoder.rs:278-335), rotation
// x[i] = a cos - b sin, x[i + rd/2] = a sin + b cos
// (crates/testing/cpu/reference-ops/src/kernels.rs:217-241).
//
// Cache layout per layer: K and V each [num_pages, nkv, page_size, d]; the page of
// position p of sequence s is block_table[s, p / page_size].
#include "common.cuh"

using namespace ilb;

constexpr int kWarpsPerBlock = 4;

template <typename TQ, typename TC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qk_norm_rope_kernel(const TQ* __restrict__ qkv, TQ* __restrict__ q_out,
                    const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                    float eps, const float2* __restrict__ rope_table, int rotary_dim,
                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                    const int* __restrict__ block_table, int max_blocks, int page_size,
                    int num_pages, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                    int n_tokens, int nq, int nkv, int d, int qkv_stride, int q_out_stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * kWarpsPerBlock + warp;
  const int total_heads = nq + 2 * nkv;
  if (head >= total_heads) return;
  float* vec = smem + warp * d;
  const TQ* src = qkv + (size_t)t * qkv_stride + (size_t)head * d;
  const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;

  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = to_float(src[i]);
    vec[i] = v;
    ss = fmaf(v, v, ss);
  }
  const float* weight = is_q ? q_weight : (is_k ? k_weight : nullptr);
  if (weight != nullptr) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    __syncwarp();
    for (int i = lane; i < d; i += 32) vec[i] = vec[i] * inv * weight[i];
  }
  __syncwarp();
  if ((is_q || is_k) && rope_table != nullptr) {
    const int half = rotary_dim / 2;
    const float2* cs = rope_table + (size_t)t * half;
    for (int i = lane; i < half; i += 32) {
      const float a = vec[i], b = vec[i + half];
      const float2 c = cs[i];
      // Products and sums rounded separately, as the reference's scalar code does.
      vec[i] = __fsub_rn(__fmul_rn(a, c.x), __fmul_rn(b, c.y));
      vec[i + half] = __fadd_rn(__fmul_rn(a, c.y), __fmul_rn(b, c.x));
    }
    __syncwarp();
  }
  if (is_q) {
    TQ* dst = q_out + (size_t)t * q_out_stride + (size_t)head * d;
    for (int i = lane; i < d; i += 32) dst[i] = from_float<TQ>(vec[i]);
    return;
  }
  if (k_cache == nullptr) return;
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  const int blk = pos / page_size;
  if (blk < 0 || blk >= max_blocks) return;
  const int page = block_table[(size_t)seq * max_blocks + blk];
  if (page < 0 || page >= num_pages) return;   // never write outside the pool
  const int kvh = is_k ? head - nq : head - nq - nkv;
  TC* dst = (is_k ? k_cache : v_cache) +
            (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * d;
  for (int i = lane; i < d; i += 32) dst[i] = from_float<TC>(vec[i]);
}

// The common geometry, bfloat16 throughout, head size 128, rotation over the whole head: one
// CTA per token, a warp takes every 8th head, a lane holds elements 2l, 2l+1 of each half of
// the head (the two members of its rotation pairs) in registers: 4-byte accesses, no shared
// memory, the loads of three heads in flight together.
constexpr int kFastWarps = 8;
constexpr int kFastUnroll = 3;

__global__ void __launch_bounds__(kFastWarps * 32)
qk_norm_rope_d128_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                         const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                         const float2* __restrict__ rope_table, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_blocks,
                         int page_size, int num_pages, __nv_bfloat16* __restrict__ k_cache,
                         __nv_bfloat16* __restrict__ v_cache, int nq, int nkv, int qkv_stride, int q_out_stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  constexpr int d = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int total_heads = nq + 2 * nkv;
  const __nv_bfloat16* row = qkv + (size_t)t * qkv_stride;
  // where this token's key and value go: looked up by the warps that hold a k or v head only
  size_t cache_off = 0;
  int cache_state = 0;                                // 0 not looked up, 1 held, -1 no page
  auto cache_row = [&]() {
    if (cache_state == 0) {
      cache_state = -1;
      if (k_cache != nullptr) {
        const int pos = positions[t], seq = seq_of_token[t];
        const int blk = pos / page_size;
        if (blk >= 0 && blk < max_blocks) {
          const int page = block_table[(size_t)seq * max_blocks + blk];
          if (page >= 0 && page < num_pages) {        // never write outside the pool
            cache_off = ((size_t)page * nkv * page_size + (pos % page_size)) * d;
            cache_state = 1;
          }
        }
      }
    }
    return cache_state == 1;
  };
  float2 cs[2] = {make_float2(1.f, 0.f), make_float2(1.f, 0.f)};
  if (rope_table != nullptr) {
    const float4 c = *reinterpret_cast<const float4*>(rope_table + (size_t)t * (d / 2) + 2 * lane);
    cs[0] = make_float2(c.x, c.y);
    cs[1] = make_float2(c.z, c.w);
  }
  float wq[4] = {1.f, 1.f, 1.f, 1.f}, wk[4] = {1.f, 1.f, 1.f, 1.f};
  if (q_weight != nullptr) { wq[0] = q_weight[2 * lane]; wq[1] = q_weight[2 * lane + 1]; wq[2] = q_weight[64 + 2 * lane]; wq[3] = q_weight[65 + 2 * lane]; }
  if (k_weight != nullptr) { wk[0] = k_weight[2 * lane]; wk[1] = k_weight[2 * lane + 1]; wk[2] = k_weight[64 + 2 * lane]; wk[3] = k_weight[65 + 2 * lane]; }

  // the CTAs of a token (gridDim.y of them: several when the tokens are few) deal its heads out warp by warp
  const int stride = kFastWarps * gridDim.y;
  for (int h0 = blockIdx.y * kFastWarps + warp; h0 < total_heads; h0 += stride * kFastUnroll) {
    uint32_t raw[kFastUnroll][2];
#pragma unroll
    for (int u = 0; u < kFastUnroll; ++u) {
      const int head = h0 + u * stride;
      if (head < total_heads) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(row + (size_t)head * d);
        raw[u][0] = src[lane];
        raw[u][1] = src[32 + lane];
      }
    }
#pragma unroll
    for (int u = 0; u < kFastUnroll; ++u) {
      const int head = h0 + u * stride;
      if (head >= total_heads) continue;                        // uniform over the warp
      const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
      const __nv_bfloat162 lo2 = *reinterpret_cast<const __nv_bfloat162*>(&raw[u][0]);
      const __nv_bfloat162 hi2 = *reinterpret_cast<const __nv_bfloat162*>(&raw[u][1]);
      float x[4] = {__low2float(lo2), __high2float(lo2), __low2float(hi2), __high2float(hi2)};
      const float* w = is_q ? (q_weight ? wq : nullptr) : (is_k ? (k_weight ? wk : nullptr) : nullptr);
      if (w != nullptr) {
        float ss = fmaf(x[0], x[0], 0.f);
        ss = fmaf(x[1], x[1], ss); ss = fmaf(x[2], x[2], ss); ss = fmaf(x[3], x[3], ss);
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = x[i] * inv * w[i];
      }
      if ((is_q || is_k) && rope_table != nullptr) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float a = x[i], b = x[2 + i];
          // Products and sums rounded separately, as the reference's scalar code does.
          x[i] = __fsub_rn(__fmul_rn(a, cs[i].x), __fmul_rn(b, cs[i].y));
          x[2 + i] = __fadd_rn(__fmul_rn(a, cs[i].y), __fmul_rn(b, cs[i].x));
        }
      }
      __nv_bfloat16* dst;
      if (is_q) dst = q_out + (size_t)t * q_out_stride + (size_t)head * d;
      else {
        if (!cache_row()) continue;
        dst = (is_k ? k_cache : v_cache) + cache_off + (size_t)(is_k ? head - nq : head - nq - nkv) * page_size * d;
      }
      __nv_bfloat162 o0 = __floats2bfloat162_rn(x[0], x[1]), o1 = __floats2bfloat162_rn(x[2], x[3]);
      reinterpret_cast<uint32_t*>(dst)[lane] = *reinterpret_cast<uint32_t*>(&o0);
      reinterpret_cast<uint32_t*>(dst)[32 + lane] = *reinterpret_cast<uint32_t*>(&o1);
    }
  }
}

// dtype: element type of qkv and q_out; cache_dtype: element type of the cache.
// q_weight / k_weight may be null (no per-head norm); rope_table may be null (no
// rotation); k_cache / v_cache may be null (this layer does not write a cache).
ILB_EXPORT int ilb_qk_norm_rope_cache(
    const void* qkv, void* q_out, int dtype, const float* q_weight, const float* k_weight,
    float eps, const float* rope_table, int rotary_dim, const int* positions,
    const int* seq_of_token, const int* block_table, int max_blocks, int page_size,
    int num_pages, void* k_cache, void* v_cache, int cache_dtype, int n_tokens, int nq, int nkv,
    int d, int qkv_stride, int q_out_stride, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && nq > 0 && nkv > 0 && d > 0, "qk_norm_rope: bad sizes");
  ILB_REQUIRE(d <= 1024, "qk_norm_rope: head size %d exceeds 1024", d);
  ILB_REQUIRE(rope_table == nullptr || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= d),
              "qk_norm_rope: rotary dimension %d must be even and at most the head size %d",
              rotary_dim, d);
  ILB_REQUIRE(qkv_stride >= (nq + 2 * nkv) * d && q_out_stride >= nq * d,
              "qk_norm_rope: strides too small");
  ILB_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "qk_norm_rope: need both caches or none");
  ILB_REQUIRE(k_cache == nullptr || (page_size > 0 && max_blocks > 0 && num_pages > 0),
              "qk_norm_rope: bad cache geometry");
  ILB_REQUIRE(dtype == cache_dtype || k_cache == nullptr || (dtype == kF32 && cache_dtype == kBF16) ||
              (dtype == kBF16 && cache_dtype == kF32), "qk_norm_rope: unknown dtypes");
  if (n_tokens == 0) return 0;
  if (dtype == kBF16 && (cache_dtype == kBF16 || k_cache == nullptr) && d == 128 && (rope_table == nullptr || rotary_dim == d) &&
      qkv_stride % 2 == 0 && q_out_stride % 2 == 0 && ((uintptr_t)qkv % 4 == 0) && ((uintptr_t)q_out % 4 == 0) &&
      ((uintptr_t)k_cache % 4 == 0) && ((uintptr_t)v_cache % 4 == 0) && ((uintptr_t)rope_table % 16 == 0)) {
    const int per_token = (nq + 2 * nkv + kFastWarps - 1) / kFastWarps;      // CTAs that give every warp one head
    int ny = 1;
    while (ny < per_token && (long long)n_tokens * ny < 592) ++ny;
    ilb::launch(qk_norm_rope_d128_kernel, dim3(n_tokens, ny), dim3(kFastWarps * 32), 0, stream,
                (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, q_weight, k_weight, eps, (const float2*)rope_table,
                positions, seq_of_token, block_table, max_blocks, page_size, num_pages, (__nv_bfloat16*)k_cache,
                (__nv_bfloat16*)v_cache, nq, nkv, qkv_stride, q_out_stride);
    return check_launch("qk_norm_rope_cache");
  }
  dim3 grid(n_tokens, (nq + 2 * nkv + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const size_t smem = (size_t)kWarpsPerBlock * d * sizeof(float);
#define ILB_LAUNCH(TQ, TC)                                                                   \
  ilb::launch(qk_norm_rope_kernel<TQ, TC>, dim3(grid), dim3(kWarpsPerBlock * 32), smem, stream,                    \
      (const TQ*)qkv, (TQ*)q_out, q_weight, k_weight, eps, (const float2*)rope_table,         \
      rotary_dim, positions, seq_of_token, block_table, max_blocks, page_size, num_pages,     \
      (TC*)k_cache, (TC*)v_cache, n_tokens, nq, nkv, d, qkv_stride, q_out_stride)
  if (dtype == kF32 && cache_dtype == kF32) ILB_LAUNCH(float, float);
  else if (dtype == kBF16 && cache_dtype == kBF16) ILB_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == kF32 && cache_dtype == kBF16) ILB_LAUNCH(float, __nv_bfloat16);
  else if (dtype == kBF16 && cache_dtype == kF32) ILB_LAUNCH(__nv_bfloat16, float);
  else return fail("qk_norm_rope: unsupported dtypes %d/%d", dtype, cache_dtype);
#undef ILB_LAUNCH
  return check_launch("qk_norm_rope_cache");
}

ILB_DEFINE_LAST_ERROR()
