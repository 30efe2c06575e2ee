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
// CTA per token; eight lanes take a head, a lane holding elements 8l .. 8l+7 of each half of
// the head (the two members of its eight rotation pairs) in registers: 16-byte accesses, no
// shared memory, a warp works on four heads at a time and has the loads of all its heads in
// flight together (up to kFastUnroll passes).
constexpr int kFastWarps = 4;
constexpr int kFastUnroll = 3;

__device__ __forceinline__ void unpack8(const uint4& r, float* x) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(w[i] << 16); x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
__device__ __forceinline__ uint4 pack8(const float* x) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

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
  const int slot = lane >> 3, l8 = lane & 7;           // which of the warp's four heads; which eighth of each half
  const int t = blockIdx.x;
  const int total_heads = nq + 2 * nkv;
  const __nv_bfloat16* row = qkv + (size_t)t * qkv_stride;
  // the loads of all this lane's heads first
  const int stride = kFastWarps * 4 * gridDim.y;       // heads between two passes (the CTAs of a token deal its heads out four by four)
  const int h0 = (blockIdx.y * kFastWarps + warp) * 4 + slot;
  uint4 raw[kFastUnroll][2];
#pragma unroll
  for (int u = 0; u < kFastUnroll; ++u) {
    const int head = h0 + u * stride;
    if (head < total_heads) {
      const uint4* src = reinterpret_cast<const uint4*>(row + (size_t)head * d);
      raw[u][0] = __ldg(src + l8);
      raw[u][1] = __ldg(src + 8 + l8);
    } else {
      raw[u][0] = make_uint4(0u, 0u, 0u, 0u);
      raw[u][1] = raw[u][0];
    }
  }
  // where this token's key and value go: looked up by the lanes that hold a k or v head only
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
  // cos and sin of this lane's eight pairs (j, j + 64), j = 8 l8 .. 8 l8 + 7
  float2 cs[8];
  if (rope_table != nullptr) {
    const float4* c = reinterpret_cast<const float4*>(rope_table + (size_t)t * (d / 2) + 8 * l8);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(c + i);
      cs[2 * i] = make_float2(v.x, v.y);
      cs[2 * i + 1] = make_float2(v.z, v.w);
    }
  }
  auto weight8 = [&](const float* w, int half, float* out8) {      // weights of elements 64 half + 8 l8 .. + 7
    const float4 a = __ldg(reinterpret_cast<const float4*>(w + 64 * half + 8 * l8));
    const float4 b = __ldg(reinterpret_cast<const float4*>(w + 64 * half + 8 * l8) + 1);
    out8[0] = a.x; out8[1] = a.y; out8[2] = a.z; out8[3] = a.w; out8[4] = b.x; out8[5] = b.y; out8[6] = b.z; out8[7] = b.w;
  };
#pragma unroll
  for (int u = 0; u < kFastUnroll; ++u) {
    const int head = h0 + u * stride;
    const bool valid = head < total_heads;
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    float x[16];                                       // [0..7]: lower half, [8..15]: upper half
    unpack8(raw[u][0], x);
    unpack8(raw[u][1], x + 8);
    const float* w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    // (every lane takes part in the exchange; a head past the end holds zeros)
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) ss = fmaf(x[i], x[i], ss);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    if (!valid) continue;
    if (w != nullptr) {
      const float inv = 1.0f / sqrtf(ss / (float)d + eps);
      float wl[8], wh[8];
      weight8(w, 0, wl);
      weight8(w, 1, wh);
#pragma unroll
      for (int i = 0; i < 8; ++i) { x[i] = x[i] * inv * wl[i]; x[8 + i] = x[8 + i] * inv * wh[i]; }
    }
    if ((is_q || is_k) && rope_table != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a = x[i], b = x[8 + i];
        // Products and sums rounded separately, as the reference's scalar code does.
        x[i] = __fsub_rn(__fmul_rn(a, cs[i].x), __fmul_rn(b, cs[i].y));
        x[8 + i] = __fadd_rn(__fmul_rn(a, cs[i].y), __fmul_rn(b, cs[i].x));
      }
    }
    __nv_bfloat16* dst;
    if (is_q) dst = q_out + (size_t)t * q_out_stride + (size_t)head * d;
    else {
      if (!cache_row()) continue;
      dst = (is_k ? k_cache : v_cache) + cache_off + (size_t)(is_k ? head - nq : head - nq - nkv) * page_size * d;
    }
    reinterpret_cast<uint4*>(dst)[l8] = pack8(x);
    reinterpret_cast<uint4*>(dst)[8 + l8] = pack8(x + 8);
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
      qkv_stride % 8 == 0 && q_out_stride % 8 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
      ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) && ((uintptr_t)rope_table % 16 == 0) &&
      ((uintptr_t)q_weight % 16 == 0) && ((uintptr_t)k_weight % 16 == 0)) {
    // CTAs per token: one takes kFastWarps x 4 heads per pass and up to kFastUnroll passes; more
    // CTAs when the heads need them, and when the tokens are too few to fill the device
    const int heads = nq + 2 * nkv, per_pass = kFastWarps * 4;
    int ny = (heads + per_pass * kFastUnroll - 1) / (per_pass * kFastUnroll);
    const int most = (heads + per_pass - 1) / per_pass;
    while (ny < most && (long long)n_tokens * ny < 1184) ++ny;
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
