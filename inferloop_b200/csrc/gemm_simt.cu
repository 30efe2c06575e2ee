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

template <typename TA, typename TO>
static int launch(const void* A, const void* W, const float* bias, void* out, int M, int N, int K,
                  int lda, int ldw, int ldo, int accumulate, cudaStream_t stream) {
  if (M <= 16) {
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
