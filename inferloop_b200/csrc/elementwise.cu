// Row-wise and element-wise kernels: embedding gather, RMSNorm, SwiGLU product,
// row gather and the rotation table.  All arithmetic is in 32-bit (the rotation
// angle in 64-bit); bfloat16 appears only as a storage type of inputs or outputs.
//
// Formulas (reference, by path within its project):
//   RMSNorm  x / sqrt(mean(x^2) + eps) * w   crates/testing/cpu/reference-ops/src/kernels.rs:38-54
//   SiLU     x * sigmoid(x), two-branch sigmoid  kernels.rs:12-22
//   RoPE     angle_i = pos / theta^(2i/rd)       kernels.rs:217-241
#include "common.cuh"

using namespace ilb;

// ---------------------------------------------------------------- embedding gather
template <typename TT>
__global__ void embed_kernel(const int* __restrict__ tokens, const TT* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  const TT* row = table + (size_t)(ok ? tok : 0) * hidden;
  float* o = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_float(row[i]) : 0.f;
}

ILB_EXPORT int ilb_embed(const int* tokens, const void* table, int table_dtype, float* out,
                         int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && hidden > 0 && vocab > 0, "embed: bad sizes T=%d H=%d V=%d",
              n_tokens, hidden, vocab);
  if (n_tokens == 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == kF32)
    ilb::launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, out, hidden, vocab);
  else if (table_dtype == kBF16)
    ilb::launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, out, hidden, vocab);
  else
    return fail("embed: unknown table dtype %d", table_dtype);
  return check_launch("embed");
}

// ---------------------------------------------------------------- RMSNorm
// One block per row.  The block size depends on the width alone, so the order of the
// additions for a row never depends on how many rows the launch holds.  A row of up to
// 4 * 1024 * kVec elements is read once with 16-byte loads and kept in registers.
constexpr int kVec = 2;                 // float4 loads per thread

template <typename TO>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                   int width, float eps) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  const float4* row = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * width);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const int n4 = width / 4;
  float4 v[kVec], g[kVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int j = threadIdx.x + i * blockDim.x;
    v[i] = j < n4 ? row[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    g[i] = j < n4 ? w4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  TO* o = out + (size_t)blockIdx.x * width;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int j = threadIdx.x + i * blockDim.x;
    if (j >= n4) continue;
    const float a = v[i].x * inv * g[i].x, b = v[i].y * inv * g[i].y;
    const float c = v[i].z * inv * g[i].z, d = v[i].w * inv * g[i].w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(o)[j] = make_float4(a, b, c, d);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(o)[j] = pk;
    }
  }
}

template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               TO* __restrict__ out, int width, float eps) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float scratch[33];
  const float* row = x + (size_t)blockIdx.x * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = row[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  TO* o = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = from_float<TO>(row[i] * inv * w[i]);
}

static inline int norm_threads(int width) {
  if (width >= 2048) return 256;
  if (width >= 512) return 128;
  if (width >= 128) return 64;
  return 32;
}

ILB_EXPORT int ilb_rmsnorm(const float* x, const float* w, void* out, int out_dtype, int rows,
                           int width, float eps, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
  ILB_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
  ILB_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "rmsnorm: unknown output dtype %d", out_dtype);
  if (rows == 0) return 0;
  const bool vec = width % 4 == 0 && width >= 1024 && width <= 4 * 1024 * kVec &&
                   ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (vec) {
    // threads = width / (4 * kVec) rounded up to a warp: the row is read exactly once
    int threads = (width / 4 + kVec - 1) / kVec;
    threads = (threads + 31) / 32 * 32;
    if (out_dtype == kF32)
      ilb::launch(rmsnorm_vec_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, w, (float*)out, width, eps);
    else
      ilb::launch(rmsnorm_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, w, (__nv_bfloat16*)out, width, eps);
    return check_launch("rmsnorm");
  }
  const int threads = norm_threads(width);
  if (out_dtype == kF32)
    ilb::launch(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, w, (float*)out, width, eps);
  else
    ilb::launch(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, w, (__nv_bfloat16*)out, width, eps);
  return check_launch("rmsnorm");
}

// ---------------------------------------------------------------- SwiGLU product
__device__ __forceinline__ float sigmoid_stable(float x) {
  if (x >= 0.f) return 1.0f / (1.0f + expf(-x));
  const float e = expf(x);
  return e / (1.0f + e);
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                T* __restrict__ out, int rows, int width, int in_stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const size_t n = (size_t)rows * width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    const float g = to_float(gate[(size_t)r * in_stride + c]);
    const float u = to_float(up[(size_t)r * in_stride + c]);
    out[i] = from_float<T>(g * sigmoid_stable(g) * u);
  }
}

// Eight bfloat16 elements per thread with 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                       __nv_bfloat16* __restrict__ out, int rows, int width8, int in_stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const size_t n = (size_t)rows * width8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / width8), c = (int)(i % width8) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate + (size_t)r * in_stride + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(up + (size_t)r * in_stride + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      o2[j] = __floats2bfloat162_rn(g.x * sigmoid_stable(g.x) * u.x, g.y * sigmoid_stable(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * width8 * 8 + c) = o4;
  }
}

// gate = in[:, 0:width], up = in[:, width:2*width] of a [rows, in_stride] matrix.
ILB_EXPORT int ilb_silu_mul(const void* in, void* out, int dtype, int rows, int width,
                            int in_stride, cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && width > 0 && in_stride >= 2 * width, "silu_mul: bad sizes");
  if (rows == 0) return 0;
  const int threads = 256;
  if (dtype == kBF16 && width % 8 == 0 && in_stride % 8 == 0 && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const size_t n8 = (size_t)rows * (width / 8);
    const int blocks8 = (int)((n8 + threads - 1) / threads < 148 * 16 ? (n8 + threads - 1) / threads : 148 * 16);
    ilb::launch(silu_mul_bf16x8_kernel, dim3(blocks8), dim3(threads), 0, stream, (const __nv_bfloat16*)in,
                (const __nv_bfloat16*)in + width, (__nv_bfloat16*)out, rows, width / 8, in_stride);
    return check_launch("silu_mul");
  }
  const size_t n = (size_t)rows * width;
  const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
  if (dtype == kF32)
    ilb::launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (const float*)in + width, (float*)out, rows, width, in_stride);
  else if (dtype == kBF16)
    ilb::launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (const __nv_bfloat16*)in + width, (__nv_bfloat16*)out, rows, width, in_stride);
  else
    return fail("silu_mul: unknown dtype %d", dtype);
  return check_launch("silu_mul");
}

// ---------------------------------------------------------------- row gather
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ idx,
                                   float* __restrict__ out, int width, int n_rows_in) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int r = idx[blockIdx.x];
  const bool ok = r >= 0 && r < n_rows_in;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[(size_t)blockIdx.x * width + i] = ok ? x[(size_t)r * width + i] : 0.f;
}

ILB_EXPORT int ilb_gather_rows(const float* x, const int* idx, float* out, int n_out, int width,
                               int n_rows_in, cudaStream_t stream) {
  ILB_REQUIRE(n_out >= 0 && width > 0, "gather_rows: bad sizes");
  if (n_out == 0) return 0;
  ilb::launch(gather_rows_kernel, dim3(n_out), dim3(256), 0, stream, x, idx, out, width, n_rows_in);
  return check_launch("gather_rows");
}

// ---------------------------------------------------------------- rotation table
// cos/sin of pos * inv_freq[i], angle and functions evaluated in 64-bit and rounded once
// to 32-bit, so the table is as good as a 32-bit number can be at any position.
__global__ void rope_table_kernel(const int* __restrict__ positions,
                                  const double* __restrict__ inv_freq,
                                  float2* __restrict__ table, int n_tokens, int half) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * half) return;
  const int t = i / half, f = i % half;
  const double angle = (double)positions[t] * inv_freq[f];
  double s, c;
  sincos(angle, &s, &c);
  table[i] = make_float2((float)c, (float)s);
}

ILB_EXPORT int ilb_rope_table(const int* positions, const double* inv_freq, float* table,
                              int n_tokens, int half, cudaStream_t stream) {
  ILB_REQUIRE(n_tokens >= 0 && half > 0, "rope_table: bad sizes");
  if (n_tokens == 0) return 0;
  const int n = n_tokens * half;
  ilb::launch(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, positions, inv_freq, (float2*)table, n_tokens, half);
  return check_launch("rope_table");
}

// ---------------------------------------------------------------- x += y (32-bit)
__global__ void add_inplace_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    x[i] += y[i];
}

ILB_EXPORT int ilb_add_inplace(float* x, const float* y, long long n, cudaStream_t stream) {
  ILB_REQUIRE(n >= 0, "add_inplace: bad size");
  if (n == 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ilb::launch(add_inplace_kernel, dim3((int)blocks), dim3(threads), 0, stream, x, y, (size_t)n);
  return check_launch("add_inplace");
}

// ---------------------------------------------------------------- x *= s, and the soft cap c * tanh(x / c) (32-bit)
// Two element-wise maps a model description may ask for: a multiplier on the embedding rows
// and a cap on the logits.  cap = 0 means "scale only".
__global__ void scale_cap_inplace_kernel(float* __restrict__ x, float scale, float cap, size_t n) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

ILB_EXPORT int ilb_scale_cap_inplace(float* x, float scale, float cap, long long n, cudaStream_t stream) {
  ILB_REQUIRE(n >= 0 && cap >= 0.f, "scale_cap_inplace: bad arguments");
  if (n == 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ilb::launch(scale_cap_inplace_kernel, dim3((int)blocks), dim3(threads), 0, stream, x, scale, cap, (size_t)n);
  return check_launch("scale_cap_inplace");
}

// ---------------------------------------------------------------- decode feedback
// After a decode step drew one token per sequence: make the next step's inputs on the
// device (token <- drawn id, position and cache length advance by one), so that a run of
// decode steps needs no host round trip.
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ positions,
                                      int* __restrict__ kv_len, const int* __restrict__ drawn,
                                      int n_live, int n) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (i < n_live) {
    tokens[i] = drawn[i];
    positions[i] += 1;
    kv_len[i] += 1;
  }
}

ILB_EXPORT int ilb_decode_advance(int* tokens, int* positions, int* kv_len, const int* drawn,
                                  int n_live, int n, cudaStream_t stream) {
  ILB_REQUIRE(n >= 0 && n_live >= 0 && n_live <= n, "decode_advance: bad sizes");
  if (n == 0) return 0;
  ilb::launch(decode_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, positions, kv_len, drawn, n_live, n);
  return check_launch("decode_advance");
}

ILB_DEFINE_LAST_ERROR()
