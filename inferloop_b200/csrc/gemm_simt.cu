// out[M,N] (+)= A[M,K] * W[N,K]^T (+ bias[N]) on the ordinary 32-bit pipes.
//
// This is the exact path: every product and sum is an IEEE 32-bit operation, no tensor-core
// mode is involved.  Each output element is summed the same way whatever the tile shape, so a
// row of A gives bit-identical results whatever other rows share the launch: blocks of 16
// consecutive k are each one chain of fused multiply-adds from zero, and the block sums are
// added in increasing order with the rounding error of every addition carried along in a
// second 32-bit word (Knuth's two-sum) and added at the end.  A plain chain over K = 12288
// terms loses about sqrt(K) units in the last place; this one stays near sqrt(16).
// With bfloat16 inputs it doubles as the any-shape fallback of the bfloat16 path.
//
// Reference formula: y = W x, weights stored [out, in]
// (crates/testing/cpu/reference-ops/src/kernels.rs:168-183).
#include "common.cuh"

using namespace ilb;

template <typename TA, typename TO, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W,
                 const float* __restrict__ bias, TO* __restrict__ out, int M, int N, int K,
                 int lda, int ldw, int ldo, int accumulate) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  constexpr int BK = 16;
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN], lost[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) { acc[i][j] = 0.f; lost[i][j] = 0.f; }

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += THREADS) {
      const int m = idx / BK, k = idx % BK;
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
    }
    for (int idx = tid; idx < BN * BK; idx += THREADS) {
      const int n = idx / BK, k = idx % BK;
      const int gn = n0 + n, gk = k0 + k;
      Ws[k][n] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
    const int kmax = (K - k0) < BK ? (K - k0) : BK;
    float part[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) part[i][j] = 0.f;
    for (int kk = 0; kk < kmax; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const float s = __fadd_rn(acc[i][j], part[i][j]);
        const float bp = __fsub_rn(s, acc[i][j]);
        lost[i][j] = __fadd_rn(lost[i][j], __fadd_rn(__fsub_rn(acc[i][j], __fsub_rn(s, bp)), __fsub_rn(part[i][j], bp)));
        acc[i][j] = s;
      }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = __fadd_rn(acc[i][j], lost[i][j]);
      if (bias != nullptr) v += bias[gn];
      TO* o = out + (size_t)gm * ldo + gn;
      if (accumulate) v = to_float(*o) + v;
      *o = from_float<TO>(v);
    }
  }
}

// The same sums, faster: operands come in 16-byte pieces (four consecutive k of a row), the
// next PF K blocks are already in registers (or on their way) while one is multiplied, and
// shared memory is double-buffered (one barrier per block of 16).  The order of the sums
// forbids cutting K among CTAs, so with few tokens and a narrow output the bytes in flight
// are all the parallelism there is: that kernel keeps eight blocks ahead.  A thread's rows and columns are strided
// (row ty + i * BM/TM, column tx + j * BN/TN), so a warp reads consecutive words.  Every output is
// still the same chains of 16 and the same compensated sum in k order as in the kernel above:
// bit for bit the same result (a zero-padded tail adds +0 to a chain).  Needs K and the leading
// dimensions multiples of 4 and 16-byte (bfloat16: 8-byte) aligned bases; rows of A beyond M
// are not multiplied by warps that hold none (a warp is one ty when BN / TN = 32).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = __ldg(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void get(float (&f)[4]) const { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
};
template <> struct Vec4<__nv_bfloat16> {
  uint2 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = __ldg(reinterpret_cast<const uint2*>(p)); }
  __device__ __forceinline__ void zero() { v = make_uint2(0u, 0u); }
  __device__ __forceinline__ void get(float (&f)[4]) const {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
  }
};

template <typename TA, typename TO, int BM, int BN, int TM, int TN, int PF>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_fast_kernel(const TA* __restrict__ A, const TA* __restrict__ W,
                      const float* __restrict__ bias, TO* __restrict__ out, int M, int N, int K,
                      int lda, int ldw, int ldo, int accumulate) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  constexpr int BK = 16;                             // K block; PF blocks are held in registers ahead of the one in shared memory
  static_assert(PF % 2 == 0, "the shared-memory buffer of a block follows from its register slot");
  constexpr int THREADS = (BM / TM) * (BN / TN);
  constexpr int XS = BN / TN, YS = BM / TM;          // strides of a thread's columns and rows
  constexpr int VA = (BM * 4 + THREADS - 1) / THREADS, VW = (BN * 4 + THREADS - 1) / THREADS;   // 4-element pieces per thread and block
  __shared__ float As[2][BK][BM + 1];
  __shared__ float Ws[2][BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid % XS, ty = tid / XS;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const bool has_rows = m0 + ty < M;                 // (rows ty + i * YS: if the first is outside, all are)
  float acc[TM][TN], lost[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) { acc[i][j] = 0.f; lost[i][j] = 0.f; }

  Vec4<TA> ras[PF][VA], rws[PF][VW];                 // (slots are only ever indexed by constants: see the unrolled loop below)
  auto fetch_into = [&](Vec4<TA> (&ra)[VA], Vec4<TA> (&rw)[VW], int k0) {
#pragma unroll
    for (int i = 0; i < VA; ++i) {
      const int v = tid + i * THREADS, row = v >> 2, k = k0 + (v & 3) * 4;
      if (v < BM * 4 && m0 + row < M && k < K) ra[i].load(A + (size_t)(m0 + row) * lda + k); else ra[i].zero();
    }
#pragma unroll
    for (int i = 0; i < VW; ++i) {
      const int v = tid + i * THREADS, row = v >> 2, k = k0 + (v & 3) * 4;
      if (v < BN * 4 && n0 + row < N && k < K) rw[i].load(W + (size_t)(n0 + row) * ldw + k); else rw[i].zero();
    }
  };
  auto stash_from = [&](const Vec4<TA> (&ra)[VA], const Vec4<TA> (&rw)[VW], int buf) {   // into shared memory, transposed
#pragma unroll
    for (int i = 0; i < VA; ++i) {
      const int v = tid + i * THREADS, row = v >> 2, k = (v & 3) * 4;
      if (v < BM * 4) {
        float f[4];
        ra[i].get(f);
#pragma unroll
        for (int j = 0; j < 4; ++j) As[buf][k + j][row] = f[j];
      }
    }
#pragma unroll
    for (int i = 0; i < VW; ++i) {
      const int v = tid + i * THREADS, row = v >> 2, k = (v & 3) * 4;
      if (v < BN * 4) {
        float f[4];
        rw[i].get(f);
#pragma unroll
        for (int j = 0; j < 4; ++j) Ws[buf][k + j][row] = f[j];
      }
    }
  };
  const int blocks = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < PF; ++s)
    if (s < blocks) fetch_into(ras[s], rws[s], s * BK);
  stash_from(ras[0], rws[0], 0);
  __syncthreads();
  for (int b0 = 0; b0 < blocks; b0 += PF) {
#pragma unroll
   for (int s = 0; s < PF; ++s) {
    const int b = b0 + s;
    if (b >= blocks) break;
    const int buf = s & 1;                                         // = b & 1: b0 is a multiple of the even PF
    // block b is in shared memory and its slot s is free: block b + PF is requested into it
    if (b + PF < blocks) fetch_into(ras[s], rws[s], (b + PF) * BK);
    if (has_rows) {
      float part[TM][TN];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) part[i][j] = 0.f;
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float a[TM], w[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) a[i] = As[buf][kk][ty + i * YS];
#pragma unroll
        for (int j = 0; j < TN; ++j) w[j] = Ws[buf][kk][tx + j * XS];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) part[i][j] = fmaf(a[i], w[j], part[i][j]);
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          const float s = __fadd_rn(acc[i][j], part[i][j]);
          const float bp = __fsub_rn(s, acc[i][j]);
          lost[i][j] = __fadd_rn(lost[i][j], __fadd_rn(__fsub_rn(acc[i][j], __fsub_rn(s, bp)), __fsub_rn(part[i][j], bp)));
          acc[i][j] = s;
        }
    }
    if (b + 1 < blocks) stash_from(ras[(s + 1) % PF], rws[(s + 1) % PF], buf ^ 1);   // block b + 1 into the other buffer (nobody reads it now)
    __syncthreads();
   }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty + i * YS;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx + j * XS;
      if (gn >= N) continue;
      float v = __fadd_rn(acc[i][j], lost[i][j]);
      if (bias != nullptr) v += bias[gn];
      TO* o = out + (size_t)gm * ldo + gn;
      if (accumulate) v = to_float(*o) + v;
      *o = from_float<TO>(v);
    }
  }
}

template <typename TA, typename TO>
static int launch(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                  int lda, int ldw, int ldo, int accumulate, cudaStream_t stream) {
  const bool pieces = K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 &&
                      (uintptr_t)A % (4 * sizeof(TA)) == 0 && (uintptr_t)W % (4 * sizeof(TA)) == 0;
  if (pieces && M <= 16) {
    constexpr int BM = 16, BN = 64, TM = 4, TN = 2;            // 4 warps, one per group of rows ty, ty + 4, ty + 8, ty + 12
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    ilb::launch(gemm_simt_fast_kernel<TA, TO, BM, BN, TM, TN, 8>, dim3(grid), dim3((BM / TM) * (BN / TN)), 0, stream,
        (const TA*)A, (const TA*)W, bias, (TO*)out, M, N, K, lda, ldw, ldo, accumulate);
  } else if (pieces) {
    constexpr int BM = 128, BN = 128, TM = 8, TN = 8;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    ilb::launch(gemm_simt_fast_kernel<TA, TO, BM, BN, TM, TN, 2>, dim3(grid), dim3((BM / TM) * (BN / TN)), 0, stream,
        (const TA*)A, (const TA*)W, bias, (TO*)out, M, N, K, lda, ldw, ldo, accumulate);
  } else if (M <= 16) {
    constexpr int BM = 16, BN = 32, TM = 2, TN = 2;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    ilb::launch(gemm_simt_kernel<TA, TO, BM, BN, TM, TN>, dim3(grid), dim3((BM / TM) * (BN / TN)), 0, stream, 
        (const TA*)A, (const TA*)W, bias, (TO*)out, M, N, K, lda, ldw, ldo, accumulate);
  } else {
    constexpr int BM = 64, BN = 64, TM = 4, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    ilb::launch(gemm_simt_kernel<TA, TO, BM, BN, TM, TN>, dim3(grid), dim3((BM / TM) * (BN / TN)), 0, stream, 
        (const TA*)A, (const TA*)W, bias, (TO*)out, M, N, K, lda, ldw, ldo, accumulate);
  }
  return check_launch("gemm_simt");
}

// in_dtype: element type of A and W; out_dtype: element type of out.
// accumulate != 0 adds the product (and bias) to what `out` already holds.
ILB_EXPORT int ilb_gemm_simt(const void* A, const void* W, const float* bias, void* out,
                             int in_dtype, int out_dtype, int M, int N, int K, int lda, int ldw,
                             int ldo, int accumulate, cudaStream_t stream) {
  ILB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  ILB_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_simt: leading dimensions too small");
  ILB_REQUIRE((long long)((N + 31) / 32) <= 2147483647LL && (M + 15) / 16 <= 65535,
              "gemm_simt: grid too large for M=%d", M);
  if (M == 0) return 0;
  if (in_dtype == kF32 && out_dtype == kF32)
    return launch<float, float>(A, W, bias, out, M, N, K, lda, ldw, ldo, accumulate, stream);
  if (in_dtype == kBF16 && out_dtype == kF32)
    return launch<__nv_bfloat16, float>(A, W, bias, out, M, N, K, lda, ldw, ldo, accumulate, stream);
  if (in_dtype == kBF16 && out_dtype == kBF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(A, W, bias, out, M, N, K, lda, ldw, ldo, accumulate, stream);
  return fail("gemm_simt: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
}

ILB_DEFINE_LAST_ERROR()
