// Token selection on the device.
//
// argmax: highest logit of a row, the lowest index among equals; a row that holds a value
// that is not finite is flagged (the reference treats it as an error:
// crates/engine/workloads/src/sampling.rs:175-192; two-stage device arg-max:
// crates/backend/cuda-kernels/src/tile/sampling/greedy_kernels.rs:17-100).
//
// sample_temperature: one draw from softmax(logits / T) by the reference's rule
// (sampling.rs:146-168, :210-226): candidates are walked from the highest logit down
// (lower index first among equals) and the first one whose cumulative normalised weight
// exceeds the uniform number u is taken.  No sort is made: the logit at which the
// cumulative weight crosses u is found by bisection on the ordered bit pattern of the
// 32-bit values (33 passes over the row), then ties at that value are walked by index.
// Weights and sums are 64-bit, as in the reference; only the ORDER of the additions
// differs, which can move the crossing point by rounding of the sums alone.
#include <math.h>
#include "common.cuh"
#include "sm100.cuh"

using namespace ilb;

constexpr int kThreads = 1024;

// Bit pattern whose unsigned order is the total order of the floats (-0 below +0).
__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// The reference's greedy rule is the total order of the values, signed zero included, lowest
// index among equals (crates/engine/workloads/src/sampling.rs:175-192).
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  const unsigned k = ordered_key(v), bk = ordered_key(bv);
  return k > bk || (k == bk && i < bi);
}

// A row is shared by the kArgmaxCtas CTAs of a thread-block cluster (contiguous parts of the
// vocabulary); each leaves its best (value, index) and its flag in shared memory, and after a
// cluster barrier CTA 0 takes the best of them from its peers' memory.  One CTA per row read
// 600 KB by itself at Qwen3's vocabulary and took 14 us.
constexpr int kArgmaxCtas = 8;

__global__ void __launch_bounds__(kThreads)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int* __restrict__ bad,
              int vocab, int stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int sbad;
  __shared__ float best_v;             // this CTA's result, read by CTA 0 of the cluster
  __shared__ int best_i, best_bad;
  const int part = blockIdx.x, n_parts = gridDim.x;
  const float* row = logits + (size_t)blockIdx.y * stride;
  const int per = (vocab + n_parts - 1) / n_parts;
  const int lo = part * per, hi = min(vocab, lo + per);
  if (threadIdx.x == 0) sbad = 0;
  __syncthreads();
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  bool nonfinite = false;
  for (int i = lo + threadIdx.x; i < hi; i += kThreads) {
    const float v = row[i];
    if (!isfinite(v)) nonfinite = true;
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
  if (nonfinite) sbad = 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = sv[lane]; bi = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { best_v = bv; best_i = bi; best_bad = sbad; }
  }
  cluster_sync_all();
  if (part == 0 && warp == 0) {
    float v = -INFINITY;
    int i = 0x7fffffff, b = 0;
    if (lane < n_parts) {
      v = ld_peer_f32(smem_u32(&best_v), (uint32_t)lane);
      i = __float_as_int(ld_peer_f32(smem_u32(&best_i), (uint32_t)lane));
      b = __float_as_int(ld_peer_f32(smem_u32(&best_bad), (uint32_t)lane));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      b |= __shfl_xor_sync(0xffffffffu, b, o);
      if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    if (lane == 0) {
      out[blockIdx.y] = i == 0x7fffffff ? 0 : i;
      if (bad != nullptr) bad[blockIdx.y] = b;
    }
  }
  cluster_sync_all();                  // nobody leaves while CTA 0 may still read its result
}

ILB_EXPORT int ilb_argmax(const float* logits, int* out, int* bad, int rows, int vocab, int stride,
                          cudaStream_t stream) {
  ILB_REQUIRE(rows >= 0 && rows <= 65535 && vocab > 0 && stride >= vocab, "argmax: bad sizes");
  if (rows == 0) return 0;
  const int parts = vocab >= 8 * kThreads ? kArgmaxCtas : 1;      // a small vocabulary is one CTA's work
  ilb::launch_cluster(argmax_kernel, dim3(parts, rows), dim3(kThreads), 0, stream, parts, logits, out, bad, vocab, stride);
  return check_launch("argmax");
}

__device__ __forceinline__ double block_sum_f64(double v, double* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double t = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__global__ void __launch_bounds__(kThreads)
sample_temperature_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                          const double* __restrict__ uniform, int* __restrict__ out,
                          int* __restrict__ bad, int vocab, int stride) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  __shared__ double scratch[33];
  __shared__ float smax[33];
  __shared__ int sflag;
  const float* row = logits + (size_t)blockIdx.x * stride;
  const double inv_t = 1.0 / (double)temperature[blockIdx.x];
  const double u = uniform[blockIdx.x];
  if (threadIdx.x == 0) sflag = 0;
  __syncthreads();
  // pass 0: maximum and finiteness
  float mx = -INFINITY;
  bool nonfinite = false;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const float v = row[i];
    if (!isfinite(v)) nonfinite = true;
    mx = fmaxf(mx, v);
  }
  if (nonfinite) sflag = 1;
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) smax[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = smax[threadIdx.x];
    t = warp_max(t);
    if (threadIdx.x == 0) smax[32] = t;
  }
  __syncthreads();
  mx = smax[32];
  if (sflag) {
    if (threadIdx.x == 0) { out[blockIdx.x] = 0; if (bad) bad[blockIdx.x] = 1; }
    return;
  }
  // pass 1: total weight
  double part = 0.0;
  for (int i = threadIdx.x; i < vocab; i += kThreads)
    part += exp(((double)row[i] - (double)mx) * inv_t);
  const double total = block_sum_f64(part, scratch);
  const double target = u * total;
  // Bisection: the largest key K such that the weight of all logits with key > K is
  // <= target; the crossing happens among the logits whose key equals the answer.
  unsigned lo = 0u, hi = ordered_key(mx);      // invariant: mass(> hi) = 0 <= target
  // mass(> key) is non-increasing in key.  Find the smallest key with mass(> key) <= target.
  while (lo < hi) {
    const unsigned mid = lo + ((hi - lo) >> 1);
    double above = 0.0;
    for (int i = threadIdx.x; i < vocab; i += kThreads) {
      const float v = row[i];
      if (ordered_key(v) > mid) above += exp(((double)v - (double)mx) * inv_t);
    }
    above = block_sum_f64(above, scratch);
    if (above <= target) hi = mid; else lo = mid + 1;
  }
  // Weight strictly above the crossing value, then walk its equals in index order.
  double above = 0.0;
  for (int i = threadIdx.x; i < vocab; i += kThreads) {
    const float v = row[i];
    if (ordered_key(v) > hi) above += exp(((double)v - (double)mx) * inv_t);
  }
  above = block_sum_f64(above, scratch);
  if (threadIdx.x == 0) {
    int chosen = -1, last = -1;
    double cumulative = above;
    for (int i = 0; i < vocab; ++i) {
      const float v = row[i];
      if (ordered_key(v) != hi) continue;
      last = i;
      cumulative += exp(((double)v - (double)mx) * inv_t);
      if (target < cumulative) { chosen = i; break; }
    }
    if (chosen < 0) chosen = last;   // rounding left the crossing past the last equal
    if (chosen < 0) {                // u at the very end: the last candidate of the walk
      float best = INFINITY; int bi = 0;
      for (int i = 0; i < vocab; ++i) if (row[i] <= best) { best = row[i]; bi = i; }
      chosen = bi;
    }
    out[blockIdx.x] = chosen;
    if (bad) bad[blockIdx.x] = 0;
  }
}

// ---------------------------------------------------------------- the same draw, shared by a cluster
// One CTA walking a row of 150,000 logits 35 times, with a 64-bit exponential per element and
// pass, took 8 to 12 ms.  Here a row belongs to a cluster of kSampleCtas CTAs (contiguous
// parts of the vocabulary).  Every thread keeps the ordered keys of its elements in registers
// and their 64-bit weights in shared memory, so a bisection pass is a compare and an add per
// element, a block sum and one exchange over the cluster's shared memory; every CTA adds the
// cluster's parts in the same order and so takes the same decisions.  The rule is the one
// above: candidates from the highest logit down, lower index first among equals, the first
// whose cumulative weight exceeds u.  Among equal logits the weights are equal, so the place
// of the crossing among them is a count, and the element at that place is found by index.
constexpr int kSampleCtas = 8;
constexpr int kSampleRegs = 24;        // elements a thread can hold: vocabularies up to 8 * 1024 * 24

__device__ __forceinline__ double ld_peer_f64(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  double v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(remote) : "memory");
  return v;
}

// Sum (or maximum) of one value per thread over the whole cluster, the same bits in every
// thread of every CTA.  `slots` [2] alternate between calls (`turn`), so that a CTA that is
// already at its next call does not overwrite what a peer still reads.
struct ClusterReduce {
  double* scratch;                     // [34]
  double* slots;                       // [2]
  int n_parts, turn;
  __device__ __forceinline__ double finish(double block_value, bool take_max) {
    if (n_parts == 1) return block_value;
    if (threadIdx.x == 0) slots[turn & 1] = block_value;
    cluster_sync_all();
    if (threadIdx.x == 0) {
      double part[kSampleCtas];
#pragma unroll
      for (int q = 0; q < kSampleCtas; ++q) part[q] = q < n_parts ? ld_peer_f64(smem_u32(slots + (turn & 1)), (uint32_t)q) : 0.0;
      double t = part[0];
#pragma unroll
      for (int q = 1; q < kSampleCtas; ++q)
        if (q < n_parts) t = take_max ? fmax(t, part[q]) : t + part[q];
      scratch[33] = t;
    }
    ++turn;
    __syncthreads();
    return scratch[33];
  }
  __device__ __forceinline__ double sum(double v) { return finish(block_sum_f64(v, scratch), false); }
  // Three sums at once (a search step looks at three keys): `wide` [3 * 33 + 3], `slots3` [2][3].
  double* wide;
  double* slots3;
  __device__ __forceinline__ void sum3(double (&v)[3]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 3; ++i) wide[i * 33 + warp] = v[i];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        double t = wide[i * 33 + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) { wide[i * 33 + 32] = t; if (n_parts > 1) slots3[(turn & 1) * 3 + i] = t; }
      }
    }
    if (n_parts > 1) {
      cluster_sync_all();
      if (threadIdx.x < 3) {                               // one thread per sum, the parts in the order of the CTAs
        double part[kSampleCtas];
#pragma unroll
        for (int q = 0; q < kSampleCtas; ++q)
          part[q] = q < n_parts ? ld_peer_f64(smem_u32(slots3 + (turn & 1) * 3 + threadIdx.x), (uint32_t)q) : 0.0;
        double t = part[0];
#pragma unroll
        for (int q = 1; q < kSampleCtas; ++q)
          if (q < n_parts) t += part[q];
        wide[99 + threadIdx.x] = t;
      }
      ++turn;
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 3; ++i) v[i] = wide[99 + i];
    } else {
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 3; ++i) v[i] = wide[i * 33 + 32];
    }
  }
  __device__ __forceinline__ double max(double v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
      double t = scratch[lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t = fmax(t, __shfl_xor_sync(0xffffffffu, t, o));
      if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return finish(scratch[32], true);
  }
};

__global__ void __launch_bounds__(kThreads)
sample_temperature_cluster_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                                  const double* __restrict__ uniform, const int* __restrict__ top_k,
                                  const float* __restrict__ top_p, const float* __restrict__ min_p,
                                  const unsigned* __restrict__ seen, const unsigned* __restrict__ generated,
                                  const float* __restrict__ repetition, const float* __restrict__ presence,
                                  int* __restrict__ out, int* __restrict__ bad, int vocab, int stride, int regs) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  extern __shared__ double weights[];                    // [regs][kThreads]
  __shared__ double scratch[34];
  __shared__ double slots[2];
  __shared__ double wide[3 * 33 + 3];
  __shared__ double slots3[6];
  const int part = blockIdx.x, n_parts = gridDim.x, t = threadIdx.x;
  const float* row = logits + (size_t)blockIdx.y * stride;
  const double inv_t = 1.0 / (double)temperature[blockIdx.y];
  const double u = uniform[blockIdx.y];
  const int per = (vocab + n_parts - 1) / n_parts;
  const int lo_i = part * per, hi_i = min(vocab, lo_i + per);
  ClusterReduce red{scratch, slots, n_parts, 0, wide, slots3};
  auto index_of = [&](int j) { return lo_i + j * kThreads + t; };

  const int words = (vocab + 31) / 32;
  const float rep = repetition ? repetition[blockIdx.y] : 1.f, pres = presence ? presence[blockIdx.y] : 0.f;
  // the row's keys into registers; maximum and finiteness
  unsigned key[kSampleRegs];
  float mx = -INFINITY;
  double nonfinite = 0.0;
#pragma unroll
  for (int j = 0; j < kSampleRegs; ++j) {
    key[j] = 0u;                                         // below every real key
    if (j < regs && index_of(j) < hi_i) {
      float v = row[index_of(j)];
      if (!isfinite(v)) nonfinite = 1.0;
      if (seen != nullptr) {
        // penalties, in 32-bit as the reference applies them: a token of the prompt or of the
        // output is scaled towards "less likely", a token of the output also loses the presence penalty
        const int i = index_of(j);
        const unsigned bit = 1u << (i & 31);
        if (seen[(size_t)blockIdx.y * words + (i >> 5)] & bit) v = v < 0.f ? v * rep : v / rep;
        if (generated[(size_t)blockIdx.y * words + (i >> 5)] & bit) v = v - pres;
      }
      mx = fmaxf(mx, v);
      key[j] = ordered_key(v);
    }
  }
  const bool any_bad = red.sum(nonfinite) > 0.0;
  if (any_bad) {                                         // (the same verdict in every CTA)
    if (part == 0 && t == 0) { out[blockIdx.y] = 0; if (bad) bad[blockIdx.y] = 1; }
    cluster_sync_all();
    return;
  }
  const double mxd = red.max((double)mx);
  auto value_of = [&](unsigned k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k); };
  // 64-bit weights, once
  double mine = 0.0;
#pragma unroll
  for (int j = 0; j < kSampleRegs; ++j)
    if (j < regs) {
      const bool on = index_of(j) < hi_i;
      const double w = on ? exp(((double)value_of(key[j]) - mxd) * inv_t) : 0.0;
      weights[j * kThreads + t] = w;
      mine += w;
    }
  const double total_all = red.sum(mine);
  auto above_key = [&](unsigned k) {                     // weight of the logits whose key is above k
    double a = 0.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (j < regs && key[j] > k) a += weights[j * kThreads + t];
    return red.sum(a);
  };
  auto count_above = [&](unsigned k) {                   // how many logits have a key above k (padding has key 0)
    double n = 0.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (j < regs && key[j] > k) n += 1.0;
    return (long long)red.sum(n);
  };
  auto equals_of = [&](unsigned k, long long& n, double& w) {   // the logits with exactly this key: how many, the weight of one
    double n_mine = 0.0, w_mine = 0.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (j < regs && key[j] == k && index_of(j) < hi_i) { n_mine += 1.0; w_mine = weights[j * kThreads + t]; }
    n = (long long)red.sum(n_mine);
    w = red.max(w_mine);
  };
  // The smallest key for which `pred(measure above the key)` holds, where the measure (a count
  // or a weight) falls as the key rises and pred holds from some key on.  A step looks at three
  // keys at once and keeps a quarter of the range: 16 steps instead of 32.
  auto search = [&](bool by_count, auto pred) {
    unsigned lo = 0u, hi = ordered_key((float)mxd);
    while (lo < hi) {
      const unsigned q2 = lo + ((hi - lo) >> 1);
      const unsigned q1 = lo + ((hi - lo) >> 2), q3 = q2 + ((hi - q2) >> 1);     // lo <= q1 <= q2 <= q3 < hi
      double a[3] = {0.0, 0.0, 0.0};
#pragma unroll
      for (int j = 0; j < kSampleRegs; ++j)
        if (j < regs) {
          const double w = by_count ? 1.0 : weights[j * kThreads + t];
          const unsigned k = key[j];
          if (k > q1) a[0] += w;
          if (k > q2) a[1] += w;
          if (k > q3) a[2] += w;
        }
      red.sum3(a);
      if (pred(a[0])) hi = q1;
      else if (pred(a[1])) { lo = q1 + 1; hi = q2; }
      else if (pred(a[2])) { lo = q2 + 1; hi = q3; }
      else lo = q3 + 1;
    }
    return hi;
  };
  // The candidates that stay are a PREFIX of the order (highest logit first, lower index first
  // among equals): everything above key `pk` and the first `pc` of its equals; (0, 0) = all.
  // top-k, min-p and top-p each name a prefix; the shortest holds.
  unsigned pk = 0u;
  long long pc = 0;
  auto shorten = [&](unsigned k, long long c) {
    if (k > pk || (k == pk && (pk == 0u || c < pc))) { pk = k; pc = c; }
  };
  const unsigned top_key = ordered_key((float)mxd);
  const int k_limit = top_k ? top_k[blockIdx.y] : 0;
  if (k_limit > 0 && k_limit < vocab) {
    const double most = (double)k_limit - 1.0;            // the smallest key with fewer than k logits above it
    const unsigned hi = search(true, [&](double n) { return n <= most; });
    shorten(hi, (long long)k_limit - count_above(hi));
  }
  const double floor_w = min_p ? (double)min_p[blockIdx.y] : 0.0;
  if (floor_w > 0.0) {
    // weights fall with the logit: the leading run with weight >= min_p ends at the lowest such key (the best always stays)
    double lowest = 4294967296.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (j < regs && index_of(j) < hi_i && (weights[j * kThreads + t] >= floor_w || key[j] == top_key))
        lowest = fmin(lowest, (double)key[j]);
    const unsigned km = (unsigned)(-red.max(-lowest));
    long long n;
    double w;
    equals_of(km, n, w);
    shorten(km, n);
  }
  auto prefix_weight = [&]() {
    if (pk == 0u) return total_all;
    long long n;
    double w;
    equals_of(pk, n, w);
    return above_key(pk) + (double)pc * w;
  };
  const double mass = top_p ? (double)top_p[blockIdx.y] : 1.0;
  if (mass < 1.0) {
    // the shortest prefix whose weight reaches mass * (weight of what stayed so far)
    const double threshold = prefix_weight() * mass;
    // the smallest key with less than the threshold above it
    const unsigned hi = search(false, [&](double a) { return a < threshold; });
    long long n;
    double w;
    equals_of(hi, n, w);
    if (n > 0) {
      const double a = above_key(hi);
      long long c = w > 0.0 ? (long long)ceil((threshold - a) / w) : n;
      c = c < 1 ? 1 : (c > n ? n : c);
      while (c > 1 && a + (double)(c - 1) * w >= threshold) --c;
      while (c < n && !(a + (double)c * w >= threshold)) ++c;
      shorten(hi, c);
    }
  }
  const double target = u * prefix_weight();
  // Bisection: the smallest key K with weight(> K) <= target; the crossing happens among the
  // logits whose key equals it.
  unsigned hi = search(false, [&](double a) { return a <= target; });
  long long n_equal, n_true;
  double w_equal;
  bool past_the_prefix = pk != 0u && hi < pk;            // the crossing lies beyond what stayed: the last that stayed
  if (past_the_prefix) hi = pk;
  const double above = above_key(hi);
  equals_of(hi, n_true, w_equal);
  n_equal = (pk != 0u && hi == pk && pc < n_true) ? pc : n_true;   // of the prefix key's equals only the first pc stayed
  // which key's equals hold the answer, and the place (1-based, by index) of the answer among them
  unsigned pick_key = hi;
  long long place = 1, count = n_true;
  if (past_the_prefix) {
    place = n_equal;
  } else if (n_equal > 0) {
    // equals weigh the same: the cumulative weight after k of them is above + k w
    long long k = w_equal > 0.0 ? (long long)floor((target - above) / w_equal) + 1 : n_equal;
    k = k < 1 ? 1 : (k > n_equal ? n_equal : k);
    while (k > 1 && target < above + (double)(k - 1) * w_equal) --k;
    while (k < n_equal && !(target < above + (double)k * w_equal)) ++k;
    place = k;                                           // never crossed: the last equal
  } else {
    // u at the very end: the last candidate of the walk, the lowest logit's highest index
    double lowest = 4294967296.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (j < regs && index_of(j) < hi_i) lowest = fmin(lowest, (double)key[j]);
    pick_key = (unsigned)(-red.max(-lowest));
    double n_mine = 0.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (j < regs && index_of(j) < hi_i && key[j] == pick_key) n_mine += 1.0;
    count = (long long)red.sum(n_mine);
    place = count;
  }
  auto is_pick = [&](int j) { return j < regs && index_of(j) < hi_i && key[j] == pick_key; };
  int chosen;
  if (place == 1 || place == count) {
    // the first or the last of the equals: one reduction over their indices
    const double sign = place == 1 ? -1.0 : 1.0;         // (one equal: both are the same element)
    double best = -4294967296.0;
#pragma unroll
    for (int j = 0; j < kSampleRegs; ++j)
      if (is_pick(j)) best = fmax(best, sign * (double)index_of(j));
    chosen = (int)(sign * red.max(best));
  } else {
    // the smallest index with `place` equals at or below it
    int ilo = 0, ihi = vocab - 1;
    while (ilo < ihi) {
      const int mid = ilo + ((ihi - ilo) >> 1);
      double n = 0.0;
#pragma unroll
      for (int j = 0; j < kSampleRegs; ++j)
        if (is_pick(j) && index_of(j) <= mid) n += 1.0;
      if ((long long)red.sum(n) >= place) ihi = mid; else ilo = mid + 1;
    }
    chosen = ilo;
  }
  if (part == 0 && t == 0) {
    out[blockIdx.y] = chosen;
    if (bad) bad[blockIdx.y] = 0;
  }
  cluster_sync_all();                                    // nobody leaves while a peer may still read its slot
}


// Bit t of row r of `seen` for every token t of request r's prompt and output so far, of
// `generated` for those of its output: entries are (row, token, 1 if generated).
__global__ void mark_tokens_kernel(const int* __restrict__ rows, const int* __restrict__ tokens,
                                   const int* __restrict__ is_generated, int n, unsigned* __restrict__ seen,
                                   unsigned* __restrict__ generated, int words, int vocab) {
  ilb::pdl_launch_dependents();
  ilb::pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int tok = tokens[i];
  if (tok < 0 || tok >= vocab) return;                   // (the caller has checked; never write outside)
  const size_t at = (size_t)rows[i] * words + (tok >> 5);
  atomicOr(seen + at, 1u << (tok & 31));
  if (is_generated[i]) atomicOr(generated + at, 1u << (tok & 31));
}

ILB_EXPORT int ilb_mark_tokens(const int* rows, const int* tokens, const int* is_generated, int n, unsigned* seen,
                               unsigned* generated, int n_rows, int vocab, cudaStream_t stream) {
  ILB_REQUIRE(n >= 0 && n_rows > 0 && vocab > 0, "mark_tokens: bad sizes");
  if (n == 0) return 0;
  ilb::launch(mark_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, rows, tokens, is_generated, n, seen, generated,
              (vocab + 31) / 32, vocab);
  return check_launch("mark_tokens");
}

// Largest vocabulary whose draws can be filtered (top-k, top-p, min-p) on the device.
ILB_EXPORT int ilb_sample_filter_max_vocab() { return kSampleCtas * kThreads * kSampleRegs; }

// top_k [rows] (0 = no limit), top_p [rows] (1 = no limit), min_p [rows] (0 = no limit): each may be null.
// seen / generated [rows][ceil(vocab / 32)] (see ilb_mark_tokens) with repetition / presence [rows], or null: penalties.
ILB_EXPORT int ilb_sample_temperature(const float* logits, const float* temperature,
                                      const double* uniform, const int* top_k, const float* top_p,
                                      const float* min_p, const unsigned* seen, const unsigned* generated,
                                      const float* repetition, const float* presence, int* out, int* bad, int rows,
                                      int vocab, int stride, cudaStream_t stream) {
  ILB_REQUIRE((seen == nullptr) == (generated == nullptr), "sample_temperature: both token bitmaps or none");
  ILB_REQUIRE(rows >= 0 && vocab > 0 && stride >= vocab, "sample_temperature: bad sizes");
  if (rows == 0) return 0;
  const int parts = vocab >= 8 * kThreads ? kSampleCtas : 1;
  const int per = (vocab + parts - 1) / parts, regs = (per + kThreads - 1) / kThreads;
  if (regs <= kSampleRegs && rows <= 65535) {
    const size_t smem = (size_t)regs * kThreads * sizeof(double);
    static OncePerDevice once;
    if (once.first())
      cudaFuncSetAttribute(sample_temperature_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)(kSampleRegs * kThreads * sizeof(double)));
    ilb::launch_cluster(sample_temperature_cluster_kernel, dim3(parts, rows), dim3(kThreads), smem, stream, parts, logits,
                        temperature, uniform, top_k, top_p, min_p, seen, generated, repetition, presence, out, bad, vocab, stride, regs);
    return check_launch("sample_temperature");
  }
  // a vocabulary beyond what the cluster's registers hold: one CTA per row walks it (no filters there)
  ILB_REQUIRE(top_k == nullptr && top_p == nullptr && min_p == nullptr && seen == nullptr,
              "sample_temperature: filtered draws are built for vocabularies up to %d", kSampleCtas * kThreads * kSampleRegs);
  ilb::launch(sample_temperature_kernel, dim3(rows), dim3(kThreads), 0, stream, logits, temperature, uniform, out, bad,
                                                           vocab, stride);
  return check_launch("sample_temperature");
}

ILB_DEFINE_LAST_ERROR()
