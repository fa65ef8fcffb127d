// Turning logits into tokens. garuda/src/runtime/mod.rs:87-175.
#include "common.cuh"

namespace {

// f(i, row[i]) for every i < V, each thread's indices in ascending order. Rows that start on a
// 16-byte boundary are read four values at a time, several loads in flight: with one CTA per row
// these passes are bound by load latency, not by bandwidth.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int V, F f) {
  int tail = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int n4 = V >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
    // eight loads are asked for before the first value is used: f may store (to memory that the
    // compiler cannot tell from the row), and a load behind a store would wait for it
    constexpr int BATCH = 8;
    const int stride = (int)blockDim.x;
    for (int q0 = threadIdx.x; q0 < n4; q0 += BATCH * stride) {
      float4 v[BATCH];
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int q = q0 + b * stride;
        v[b] = q < n4 ? r4[q] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int q = q0 + b * stride;
        if (q < n4) {
          f(4 * q, v[b].x); f(4 * q + 1, v[b].y); f(4 * q + 2, v[b].z); f(4 * q + 3, v[b].w);
        }
      }
    }
    tail = 4 * n4;
  }
  for (int i = tail + threadIdx.x; i < V; i += blockDim.x) f(i, row[i]);
}

// Greedy: the first maximum wins (a strict `>` scan from index 0, :99-107), so
// among equal values the lowest index is kept, and NaN never wins.
__device__ int block_argmax(const float* __restrict__ row, int V) {
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for_each_logit(row, V, [&](int i, float v) {
    if (v > best) { best = v; best_i = i; }  // ascending i within a thread: first maximum
  });
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int result;
  auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    best_i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) result = best_i == 0x7fffffff ? 0 : best_i;
  }
  __syncthreads();
  return result;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int V) {
  const int tok = block_argmax(logits + (size_t)blockIdx.x * V, V);
  if (threadIdx.x == 0) out[blockIdx.x] = tok;
}

// ------------------------------------------------------------------ sampling
// Temperature, softmax over the whole vocabulary, top-k, top-p, then a draw
// (garuda/src/runtime/mod.rs:109-175). The reference sorts the candidates by
// (probability descending, token id ascending), keeps the first k, of those the
// shortest prefix whose probabilities sum to top_p, and walks that list
// subtracting probabilities from u * total until it reaches zero. Survivors are
// not renormalised.
//
// Two ways. With top_k of at most 1,024 (sample_from_top_k below) the k most likely
// tokens are found by a radix selection on the probabilities' bit patterns, sorted in
// shared memory, and walked as the reference walks them. Otherwise (no top_k, or a
// larger one) nothing is sorted: "the j-th candidate" is found by bisecting on the bit
// pattern of the probability (non-negative floats order like their bits): for a
// threshold tau one pass gives how many probabilities exceed it, how many equal
// it, and the sum of those that exceed it. Sums are taken in 64-bit so that
// their order does not matter.

struct Tally {
  int gt;      // how many p > tau
  int eq;      // how many p == tau
  double sgt;  // sum of those > tau
  float tau;
  __device__ int ge() const { return gt + eq; }
  __device__ double sge() const { return sgt + (double)eq * (double)tau; }
};

__device__ Tally block_tally(const float* __restrict__ p, int V, uint32_t tau_bits, double* sh_d, int* sh_i) {
  int gt = 0, eq = 0;
  double sgt = 0.0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = p[i];
    const uint32_t b = __float_as_uint(v);
    if (b > tau_bits) { ++gt; sgt += (double)v; }
    else if (b == tau_bits) ++eq;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    gt += __shfl_xor_sync(0xffffffffu, gt, o);
    eq += __shfl_xor_sync(0xffffffffu, eq, o);
    sgt += __shfl_xor_sync(0xffffffffu, sgt, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();  // everyone has read the previous result
  if (lane == 0) { sh_i[warp] = gt; sh_i[32 + warp] = eq; sh_d[warp] = sgt; }
  __syncthreads();
  Tally t{0, 0, 0.0, __uint_as_float(tau_bits)};
  for (int w = 0; w < nw; ++w) { t.gt += sh_i[w]; t.eq += sh_i[32 + w]; t.sgt += sh_d[w]; }
  return t;
}

// The largest tau for which pred(tally(tau)) holds. pred must hold for small
// tau and fail for large ones. Returns false if it does not even hold at 0.
template <typename Pred>
__device__ bool bisect(const float* p, int V, double* sh_d, int* sh_i, Pred pred, Tally* found) {
  Tally best = block_tally(p, V, 0u, sh_d, sh_i);
  if (!pred(best)) return false;
  uint32_t cur = 0;
  for (int bit = 30; bit >= 0; --bit) {  // probabilities lie in [0, 1]: the sign bit is never set
    const uint32_t cand = cur | (1u << bit);
    if (cand > 0x3f800000u) continue;    // above 1.0 nothing is left
    const Tally t = block_tally(p, V, cand, sh_d, sh_i);
    if (pred(t)) { cur = cand; best = t; }
  }
  *found = best;
  return true;
}

// Called by the first warp: the bin of hist[0..255] that holds the `remaining`-th value from the top
// goes to sh_i[0], its rank within that bin to sh_i[1]. Every lane sums eight bins, a suffix sum over
// the lanes finds the lane, which then walks its own eight.
__device__ __forceinline__ void pick_bin(const int* hist, int remaining, int* sh_i) {
  const int lane = threadIdx.x;
  int mine8 = 0;
#pragma unroll
  for (int q = 0; q < 8; ++q) mine8 += hist[8 * lane + q];
  int suffix = mine8;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_down_sync(0xffffffffu, suffix, o);
    if (lane + o < 32) suffix += v;
  }
  int above = suffix - mine8;                      // in the bins of the lanes above this one
  if (above < remaining && remaining <= suffix) {
    int bin = 8 * lane + 7;
    for (; bin > 8 * lane; --bin) {
      if (above + hist[bin] >= remaining) break;
      above += hist[bin];
    }
    sh_i[0] = bin;
    sh_i[1] = remaining - above;
  }
}

// top_k of at most LIST_MAX, the usual case: the k most likely tokens are picked out and sorted,
// and top-p, the total mass and the walk to the drawn point run over that short list exactly as the
// reference walks its sorted candidates (garuda/src/runtime/mod.rs:109-172), instead of one bisection
// over the whole vocabulary for each of them.
constexpr int LIST_MAX = 1024;

// keys[0 .. count): candidates as (probability bits, ~token id), among them the kk most likely ones
// by (probability descending, token id ascending). Sorts them that way and walks the first kk as the
// reference walks its sorted candidates. Every thread of the block calls it; see sample_from_top_k for
// must_reach and the result.
__device__ bool sort_and_walk(unsigned long long* keys, int count, int kk, int V, float tp, float uniform_draw,
                              int32_t* out, int* sh_i, bool must_reach) {
  // sort descending (bitonic, padded with zeros to a power of two)
  int size = 1;
  while (size < count) size <<= 1;
  for (int i = count + threadIdx.x; i < size; i += blockDim.x) keys[i] = 0ull;
  __syncthreads();
  if (size <= 64) {
    // a short list is sorted by the first warp alone: no block-wide barriers
    if (threadIdx.x < 32) {
      for (int span = 2; span <= size; span <<= 1) {
        for (int step = span >> 1; step > 0; step >>= 1) {
          for (int i = threadIdx.x; i < size; i += 32) {
            const int other = i ^ step;
            if (other > i) {
              const unsigned long long a = keys[i], b = keys[other];
              const bool descending = (i & span) == 0;
              if (descending ? a < b : a > b) { keys[i] = b; keys[other] = a; }
            }
          }
          __syncwarp();
        }
      }
    }
    __syncthreads();
  } else
  for (int span = 2; span <= size; span <<= 1) {
    for (int step = span >> 1; step > 0; step >>= 1) {
      for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const int other = i ^ step;
        if (other > i) {
          const unsigned long long a = keys[i], b = keys[other];
          const bool descending = (i & span) == 0;
          if (descending ? a < b : a > b) { keys[i] = b; keys[other] = a; }
        }
      }
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) {
    auto prob = [&](int i) { return (double)__uint_as_float((uint32_t)(keys[i] >> 32)); };
    // n: how many candidates survive top-p (:161-172) within the top k (:144-158)
    int n = kk;
    bool reached = tp >= 1.0f || kk == V;
    double mass = 0.0;                         // of the first n
    for (int i = 0; i < kk; ++i) {
      mass += prob(i);
      if (tp < 1.0f && mass >= (double)tp) { n = i + 1; reached = true; break; }
    }
    sh_i[3] = (must_reach && !reached) ? 0 : 1;
    const float total = (float)mass;
    int j = 1;    // zero mass: the most likely one (:111-115)
    if (sh_i[3] == 0) {
      // top-p reaches beyond this list: the caller goes on without it
    } else if (total > 0.f) {
      const double point = (double)(uniform_draw * total);
      double cum = 0.0;
      j = n;
      for (int i = 0; i < n; ++i) {
        cum += prob(i);
        if (cum >= point) { j = i + 1; break; }
      }
    }
    if (sh_i[3] != 0) *out = (int32_t)(0xffffffffu - (uint32_t)(keys[j - 1] & 0xffffffffull));
  }
  __syncthreads();
  const bool done = sh_i[3] != 0;
  __syncthreads();      // before sh_i is used again
  return done;
}

// p: the row's probabilities. Ends with the chosen token in *out. Every thread of the block calls it.
// must_reach: top-p has to be reached within these k (the caller has no top-k of its own and tries the k
// most likely tokens first); if it is not, nothing is written and false returned, to every thread.
__device__ bool sample_from_top_k(const float* p, int V, int k, float tp, float uniform_draw, int32_t* out,
                                  int* sh_cnt, int* sh_i, bool must_reach, unsigned long long* keys, int* hist) {
  const int kk = min(k, V);
  // the kk-th largest probability by its bit pattern, a byte at a time from the top
  uint32_t prefix = 0;
  int remaining = kk;
  for (int shift = 24; shift >= 0; shift -= 8) {
    const uint32_t mask = shift == 24 ? 0u : 0xffffffffu << (shift + 8);
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    // Probabilities crowd into a few bins (most share their exponent), so the lanes of a warp that
    // hit the same bin add to it once, together.
    const int padded = (V + 31) & ~31;
    for (int i = threadIdx.x; i < padded; i += blockDim.x) {
      const uint32_t b = i < V ? __float_as_uint(p[i]) : 0u;
      const int bin = (i < V && (b & mask) == (prefix & mask)) ? (int)((b >> shift) & 255u) : 256;
      const unsigned peers = __match_any_sync(0xffffffffu, bin);
      if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
    }
    __syncthreads();
    if (threadIdx.x < 32) pick_bin(hist, remaining, sh_i);
    __syncthreads();
    prefix |= (uint32_t)sh_i[0] << shift;
    remaining = sh_i[1];
    __syncthreads();
  }
  const uint32_t tau_bits = prefix;   // the kk-th largest; `remaining` of those equal to it are wanted
  const int gt = kk - remaining;
  if (must_reach && kk < V) {
    // Before the list is gathered, sorted and walked: does its mass reach top-p at all? (With a slack
    // for the order of the additions: a list that only just reaches it is walked and decides itself.)
    __shared__ double part[32];
    double above = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = p[i];
      if (__float_as_uint(v) > tau_bits) above += (double)v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) above += __shfl_xor_sync(0xffffffffu, above, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = above;
    __syncthreads();
    double mass = (double)remaining * (double)__uint_as_float(tau_bits);
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mass += part[w];
    __syncthreads();
    if (mass < (double)tp * (1.0 - 1e-6)) return false;
  }
  // gather: everything above tau in any order (the sort below orders it), and of those equal to tau
  // the `remaining` lowest token ids. For these every warp takes a run of the vocabulary and walks it
  // 32 tokens at a time, so that ranks among the ties follow the token ids.
  if (threadIdx.x == 0) sh_i[2] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int run = ((V + nw - 1) / nw + 31) & ~31;            // tokens per warp, whole walks of 32
  const int lo = min(V, warp * run), hi = min(V, lo + run);
  int ties = 0;
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const uint32_t b = i < hi ? __float_as_uint(p[i]) : 0u;
    if (i < hi && b > tau_bits) keys[atomicAdd(&sh_i[2], 1)] = ((unsigned long long)b << 32) | (0xffffffffu - (uint32_t)i);
    ties += __popc(__ballot_sync(0xffffffffu, i < hi && b == tau_bits));
  }
  if (lane == 0) sh_cnt[warp] = ties;
  __syncthreads();
  int before = 0;                                            // ties in the runs of the warps in front
  for (int w = 0; w < warp; ++w) before += sh_cnt[w];
  for (int base = lo; base < hi && before < remaining; base += 32) {
    const int i = base + lane;
    const bool tie = i < hi && __float_as_uint(p[i]) == tau_bits;
    const unsigned votes = __ballot_sync(0xffffffffu, tie);
    const int rank = before + __popc(votes & ((1u << lane) - 1u));
    if (tie && rank < remaining) keys[gt + rank] = ((unsigned long long)tau_bits << 32) | (0xffffffffu - (uint32_t)i);
    before += __popc(votes);
  }
  return sort_and_walk(keys, kk, kk, V, tp, uniform_draw, out, sh_i, must_reach);
}

// top_k below the number of threads, the usual case of all: no pass over the vocabulary beyond one
// that picks candidates out. Every thread knows the largest probability among its own tokens; the k-th
// largest of these maxima is a lower bound of the k-th largest probability (each of the k threads above
// it holds a token at least that likely), so every one of the k most likely tokens, and every token
// tied with the last of them, is at least that likely. Those tokens, a few more than k, are sorted and
// walked. e: the exponentials before their division by the sum (p = e * inv, as the full pass computes
// it); thread_max: the largest of the thread's own p. False, to every thread, if the candidates do not
// fit the list (many equal probabilities): the caller goes on the general way.
__device__ bool sample_from_short_list(const float* e, int V, int k, float inv, float thread_max, float tp,
                                       float uniform_draw, int32_t* out, int* sh_i, unsigned long long* keys, int* hist) {
  // the k-th largest maximum, to its upper 16 bits: a lower bound still
  uint32_t prefix = 0;
  int remaining = k;
  const uint32_t mine = __float_as_uint(thread_max);
  for (int shift = 24; shift >= 16; shift -= 8) {
    const uint32_t mask = shift == 24 ? 0u : 0xffffffffu << (shift + 8);
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    if ((mine & mask) == (prefix & mask)) atomicAdd(&hist[(mine >> shift) & 255u], 1);
    __syncthreads();
    if (threadIdx.x < 32) pick_bin(hist, remaining, sh_i);
    __syncthreads();
    prefix |= (uint32_t)sh_i[0] << shift;
    remaining = sh_i[1];
    __syncthreads();
  }
  const uint32_t bound = prefix;
  if (threadIdx.x == 0) sh_i[2] = 0;
  __syncthreads();
  // (several loads in flight: with a vocabulary too large for shared memory the exponentials lie in
  // global memory, and a loop of single loads would wait out the latency of each)
  for_each_logit(e, V, [&](int i, float v) {
    const uint32_t b = __float_as_uint(v * inv);
    if (b >= bound) {
      const int at = atomicAdd(&sh_i[2], 1);
      if (at < LIST_MAX) keys[at] = ((unsigned long long)b << 32) | (0xffffffffu - (uint32_t)i);
    }
  });
  __syncthreads();
  const int count = sh_i[2];
  __syncthreads();      // before sh_i is used again
  if (count > LIST_MAX || count < k) return false;
  return sort_and_walk(keys, count, k, V, tp, uniform_draw, out, sh_i, false);
}

// What the sampling kernels keep in shared memory beside a row's probabilities.
struct SampleShared {
  double sh_d[32];
  int sh_i[64];
  float sh_f[32];
  int sh_cnt[1024];
  unsigned long long keys[LIST_MAX];   // probability bits, then ~token id: descending = by probability, then by id
  int hist[257];                       // bin 256 takes what a pass does not count
};

// One row by one CTA: every thread of the block calls it. p: room for the row's probabilities
// (shared memory, or the caller's scratch).
__device__ void sample_row(const float* __restrict__ logits, const float* __restrict__ temperature,
                           const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
                           const float* __restrict__ u, int32_t* __restrict__ out, float* p, int V, int r,
                           SampleShared& sh) {
  double* sh_d = sh.sh_d;
  int* sh_i = sh.sh_i;
  float* sh_f = sh.sh_f;
  int* sh_cnt = sh.sh_cnt;
  unsigned long long* keys = sh.keys;
  int* hist = sh.hist;
  const float* row = logits + (size_t)r * V;
  const float temp = temperature[r];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (temp == 0.f) {  // greedy (:99-107)
    const int tok = block_argmax(row, V);
    if (threadIdx.x == 0) out[r] = tok;
    return;
  }

  // softmax(logits / temperature), with the reference's uniform fallbacks
  // (garuda/src/simd/mod.rs:132-158)
  float m = -INFINITY;
  // (the largest quotient is the quotient of the largest logit: division by a positive number is
  // monotonic, also after rounding; one division instead of one per token)
  for_each_logit(row, V, [&](int, float v) { m = fmaxf(m, v); });
  m = gb::warp_max(m);
  if (lane == 0) sh_f[warp] = m;
  __syncthreads();
  m = -INFINITY;
  for (int w = 0; w < nw; ++w) m = fmaxf(m, sh_f[w]);
  m = m / temp;
  const bool finite_max = (m - m) == 0.f;  // neither infinite nor NaN
  double sum = 0.0;
  float largest = 0.f;       // of this thread's exponentials
  for_each_logit(row, V, [&](int i, float v) {
    const float e = finite_max ? expf(v / temp - m) : 1.0f;
    p[i] = e;
    sum += (double)e;
    largest = fmaxf(largest, e);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) sh_d[warp] = sum;
  __syncthreads();
  sum = 0.0;
  for (int w = 0; w < nw; ++w) sum += sh_d[w];
  const float fsum = (float)sum;
  const bool good = finite_max && (fsum - fsum) == 0.f && fsum > 0.f;  // a NaN among the inputs fails here
  const float inv = good ? 1.0f / fsum : 0.f;
  const float uniform = 1.0f / (float)V;
  if (good && top_k[r] > 0 && top_k[r] < (int)blockDim.x && top_k[r] < V && top_k[r] <= LIST_MAX) {
    __syncthreads();          // the exponentials of all threads are in place
    if (sample_from_short_list(p, V, top_k[r], inv, largest * inv, top_p[r], u[r], out + r, sh_i, keys, hist)) return;
  }
  for (int i = threadIdx.x; i < V; i += blockDim.x) p[i] = good ? p[i] * inv : uniform;
  __syncthreads();

  if (top_k[r] > 0 && top_k[r] <= LIST_MAX) {
    sample_from_top_k(p, V, top_k[r], top_p[r], u[r], out + r, sh_cnt, sh_i, false, keys, hist);
    return;
  }
  // top-p alone (or with a top-k beyond the list): nearly always it is reached within the LIST_MAX most
  // likely tokens, and then those are all that matter
  if (top_p[r] < 1.0f && sample_from_top_k(p, V, LIST_MAX, top_p[r], u[r], out + r, sh_cnt, sh_i, true, keys, hist)) return;

  // n: how many candidates survive top-k (:144-158) and top-p (:161-172)
  int n = V;
  Tally t;
  const float tp = top_p[r];
  if (tp < 1.0f) {
    const double want = (double)tp;
    if (bisect(p, V, sh_d, sh_i, [&](const Tally& a) { return a.ge() >= 1 && a.sge() >= want; }, &t)) {
      // candidates above tau, then as many of those equal to tau as it takes to reach top_p
      int ties = t.tau > 0.f ? (int)ceil((want - t.sgt) / (double)t.tau) : t.eq;
      ties = max(1, min(ties, t.eq));
      n = t.gt + ties;
    }
  }
  const int k = top_k[r];
  if (k > 0 && k < n) n = k;

  // total mass of the first n (:109), and the point the walk has to reach (:117)
  bisect(p, V, sh_d, sh_i, [&](const Tally& a) { return a.ge() >= n; }, &t);
  const float total = (float)(t.sgt + (double)(n - t.gt) * (double)t.tau);
  int j = 1;  // 1-based rank of the chosen candidate; zero mass: the most likely one (:111-115)
  if (total > 0.f) {
    const double point = (double)(u[r] * total);
    Tally x;
    if (bisect(p, V, sh_d, sh_i, [&](const Tally& a) { return a.ge() >= 1 && a.sge() >= point; }, &x)) {
      int ties = x.tau > 0.f ? (int)ceil((point - x.sgt) / (double)x.tau) : 1;
      ties = max(1, min(ties, x.eq));
      j = x.gt + ties;
    } else {
      j = n;
    }
    j = max(1, min(j, n));
  }

  // the j-th candidate: value of the j-th largest, then by token id among equals
  bisect(p, V, sh_d, sh_i, [&](const Tally& a) { return a.ge() >= j; }, &t);
  const int want_tie = j - t.gt;  // 1-based among p == tau, ascending id
  const uint32_t tau_bits = __float_as_uint(t.tau);
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
  int mine = 0;
  for (int i = lo; i < hi; ++i) mine += (__float_as_uint(p[i]) == tau_bits);
  sh_cnt[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    int seen = 0, owner = -1, skip = 0;
    for (int th = 0; th < (int)blockDim.x; ++th) {
      if (seen + sh_cnt[th] >= want_tie) { owner = th; skip = want_tie - seen; break; }
      seen += sh_cnt[th];
    }
    sh_i[0] = owner;
    sh_i[1] = skip;
  }
  __syncthreads();
  if ((int)threadIdx.x == sh_i[0]) {
    int left = sh_i[1];
    for (int i = lo; i < hi; ++i) {
      if (__float_as_uint(p[i]) == tau_bits && --left == 0) { out[r] = i; break; }
    }
  }
}

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ u, int32_t* __restrict__ out, float* __restrict__ scratch, int V,
              int in_shared) {
  extern __shared__ float row_shared[];      // in_shared: the row's probabilities live here, not in scratch
  __shared__ SampleShared sh;
  const int r = blockIdx.x;
  sample_row(logits, temperature, top_k, top_p, u, out, in_shared ? row_shared : scratch + (size_t)r * V, V, r, sh);
}


// ------------------------------------------------------------------ a row by a cluster of CTAs
// One CTA works through a row at the pace of one SM's arithmetic: a division, an exponential and a
// handful of other instructions per token and pass (60 us at 128,256 tokens). With a small top_k
// the passes over the vocabulary are all there is to do, so the eight CTAs of a cluster take an
// eighth of the row each: the maximum and the sum are exchanged through the cluster's shared
// memory, every CTA bounds the k-th largest probability from below within its own part (see
// sample_from_short_list; the largest of the bounds holds for the whole row), and the candidates go
// straight into the first CTA's list, which sorts and walks them. Rows it does not take (greedy, no
// or a large top_k, a degenerate softmax, more candidates than the list holds) are done by the
// first CTA alone, the general way, in the caller's scratch memory.
constexpr int ROW_CTAS = 8;
constexpr int SMALL_K = 64;

__device__ __forceinline__ uint32_t shared_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t in_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __cluster_dims__(ROW_CTAS, 1, 1) __launch_bounds__(1024)
sample_cluster_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                      const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
                      const float* __restrict__ u, int32_t* __restrict__ out, float* __restrict__ scratch, int V) {
  extern __shared__ float part_e[];          // this CTA's part of the row: the exponentials
  __shared__ SampleShared sh;
  __shared__ float c_max[ROW_CTAS];
  __shared__ double c_sum[ROW_CTAS];
  __shared__ uint32_t c_bound[ROW_CTAS];
  const int r = blockIdx.x / ROW_CTAS;
  const uint32_t rank = cluster_rank();
  const float temp = temperature[r];
  const int k = top_k[r];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  // the same for every CTA of the cluster: either all go on, or the first one works alone
  if (temp == 0.f || k <= 0 || k > SMALL_K || k >= V) {
    if (rank == 0) sample_row(logits, temperature, top_k, top_p, u, out, scratch + (size_t)r * V, V, r, sh);
    return;
  }
  const float* row = logits + (size_t)r * V;
  const int per = (((V + ROW_CTAS - 1) / ROW_CTAS) + 3) & ~3;     // a multiple of four: parts start on 16 bytes if the row does
  const int lo = min(V, (int)rank * per), n = min(V, lo + per) - lo;

  // the row's maximum
  float m = -INFINITY;
  for_each_logit(row + lo, n, [&](int, float v) { m = fmaxf(m, v); });
  m = gb::warp_max(m);
  if (lane == 0) sh.sh_f[warp] = m;
  if (threadIdx.x == 0) sh.sh_i[2] = 0;            // the first CTA's count of candidates
  __syncthreads();
  if (threadIdx.x < ROW_CTAS) {
    float mine = -INFINITY;
    for (int w = 0; w < nw; ++w) mine = fmaxf(mine, sh.sh_f[w]);
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(in_rank(shared_u32(&c_max[rank]), threadIdx.x)), "f"(mine) : "memory");
  }
  cluster_sync_all();
  m = -INFINITY;
  for (int c = 0; c < ROW_CTAS; ++c) m = fmaxf(m, c_max[c]);
  m = m / temp;
  const bool finite_max = (m - m) == 0.f;

  // exponentials of this part, their sum, every thread's largest
  double sum = 0.0;
  float largest = 0.f;
  for_each_logit(row + lo, n, [&](int i, float v) {
    const float e = finite_max ? expf(v / temp - m) : 1.0f;
    part_e[i] = e;
    sum += (double)e;
    largest = fmaxf(largest, e);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) sh.sh_d[warp] = sum;
  __syncthreads();
  // the k-th largest of the threads' maxima, to its upper 16 bits: at least k tokens of this part are
  // at least that likely
  uint32_t prefix = 0;
  {
    int remaining = k;
    const uint32_t mine = __float_as_uint(largest);
    for (int shift = 24; shift >= 16; shift -= 8) {
      const uint32_t mask = shift == 24 ? 0u : 0xffffffffu << (shift + 8);
      if (threadIdx.x < 256) sh.hist[threadIdx.x] = 0;
      __syncthreads();
      if ((mine & mask) == (prefix & mask)) atomicAdd(&sh.hist[(mine >> shift) & 255u], 1);
      __syncthreads();
      if (threadIdx.x < 32) pick_bin(sh.hist, remaining, sh.sh_i);
      __syncthreads();
      prefix |= (uint32_t)sh.sh_i[0] << shift;
      remaining = sh.sh_i[1];
      __syncthreads();
    }
  }
  if (threadIdx.x < ROW_CTAS) {
    double mine = 0.0;
    for (int w = 0; w < nw; ++w) mine += sh.sh_d[w];
    asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(in_rank(shared_u32(&c_sum[rank]), threadIdx.x)), "d"(mine) : "memory");
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(in_rank(shared_u32(&c_bound[rank]), threadIdx.x)), "r"(prefix) : "memory");
  }
  cluster_sync_all();
  double total = 0.0;
  uint32_t bound_e = 0;
  for (int c = 0; c < ROW_CTAS; ++c) {
    total += c_sum[c];
    bound_e = max(bound_e, c_bound[c]);
  }
  const float fsum = (float)total;
  const bool good = finite_max && (fsum - fsum) == 0.f && fsum > 0.f;
  if (!good) {          // the same verdict in every CTA
    if (rank == 0) sample_row(logits, temperature, top_k, top_p, u, out, scratch + (size_t)r * V, V, r, sh);
    return;
  }
  const float inv = 1.0f / fsum;
  // e >= bound implies e * inv >= bound * inv (rounding keeps the order)
  const uint32_t bound = __float_as_uint(__uint_as_float(bound_e) * inv);
  const uint32_t count_at = in_rank(shared_u32(&sh.sh_i[2]), 0), keys_at = in_rank(shared_u32(&sh.keys[0]), 0);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t b = __float_as_uint(part_e[i] * inv);
    if (b >= bound) {
      uint32_t at;
      asm volatile("atom.shared::cluster.add.u32 %0, [%1], 1;" : "=r"(at) : "r"(count_at) : "memory");
      if (at < (uint32_t)LIST_MAX) {
        const unsigned long long key = ((unsigned long long)b << 32) | (0xffffffffu - (uint32_t)(lo + i));
        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(keys_at + at * 8u), "l"(key) : "memory");
      }
    }
  }
  cluster_sync_all();
  if (rank != 0) return;
  const int count = sh.sh_i[2];
  __syncthreads();      // before sh_i is used again
  if (count > LIST_MAX || count < k) {       // many equal probabilities: the general way
    sample_row(logits, temperature, top_k, top_p, u, out, scratch + (size_t)r * V, V, r, sh);
    return;
  }
  sort_and_walk(sh.keys, count, k, V, top_p[r], u[r], out + r, sh.sh_i, false);
}

}  // namespace


GB_EXPORT int gb_argmax(const float* logits, int32_t* out, int R, int V, cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  if (V <= 0) return gb::fail(GB_BAD_ARGUMENT, "cannot sample from empty logits");
  argmax_kernel<<<R, 1024, 0, stream>>>(logits, out, V);
  return gb::check_launch("argmax");
}

namespace {
// A row's probabilities are read a dozen times (hundreds without a small top_k): they are kept in
// shared memory when the vocabulary fits there (about 50,000 tokens), else in `scratch`.
int launch_sample(const float* logits, const float* temperature, const int32_t* top_k, const float* top_p,
                  const float* u, int32_t* out, float* scratch, int R, int V, cudaStream_t stream) {
  constexpr size_t LIMIT = 200 * 1024;
  const size_t bytes = (size_t)V * sizeof(float);
  const bool fits = bytes <= LIMIT;
  static gb::OncePerDevice configured;
  if (fits && configured.needed()) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LIMIT);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "sample: %s", cudaGetErrorString(e));
    configured.done();
  }
  sample_kernel<<<R, 1024, fits ? bytes : 0, stream>>>(logits, temperature, top_k, top_p, u, out, scratch, V,
                                                       fits ? 1 : 0);
  return gb::check_launch("sample");
}
}  // namespace

// The same where every row is greedy or has a top_k of at most 64: eight CTAs share a row's passes
// over the vocabulary (other rows are still right, only slower than through gb_sample).
GB_EXPORT int gb_sample_small_k(const float* logits, const float* temperature, const int32_t* top_k,
                                const float* top_p, const float* u, int32_t* out, float* scratch, int R, int V,
                                cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  if (V <= 0) return gb::fail(GB_BAD_ARGUMENT, "cannot sample from empty logits");
  const int per = (((V + ROW_CTAS - 1) / ROW_CTAS) + 3) & ~3;
  const size_t bytes = (size_t)per * sizeof(float);
  // more rows than the SMs hold clusters of: one CTA per row is as fast (measured: 64 rows)
  static int sms = [] {
    int dev = 0, v = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v;
  }();
  if (bytes > 160 * 1024 || R * ROW_CTAS > sms)
    return launch_sample(logits, temperature, top_k, top_p, u, out, scratch, R, V, stream);
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "sample: %s", cudaGetErrorString(e));
    configured.done();
  }
  sample_cluster_kernel<<<R * ROW_CTAS, 1024, bytes, stream>>>(logits, temperature, top_k, top_p, u, out, scratch, V);
  return gb::check_launch("sample (clusters)");
}

// One token per row of logits [R, V]. Rows with temperature 0 are greedy.
// scratch: R * V floats of work space (the probabilities, where a row does not fit in shared memory).
GB_EXPORT int gb_sample(const float* logits, const float* temperature, const int32_t* top_k,
                        const float* top_p, const float* u, int32_t* out, float* scratch, int R, int V,
                        cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  if (V <= 0) return gb::fail(GB_BAD_ARGUMENT, "cannot sample from empty logits");
  return launch_sample(logits, temperature, top_k, top_p, u, out, scratch, R, V, stream);
}

// ---------------------------------------------------------------------------
// gb_sample_noalloc: the same kernel with work space that the library brings
// itself, for callers that cannot allocate (see no_alloc.h for the contract).
#include "no_alloc.h"

namespace {

// The work space. In host code this name is only a handle for the runtime's
// symbol calls, never an address a kernel could use; the device address is
// looked up once per device below.
static __device__ __align__(256) float g_noalloc_scratch[GB_SAMPLE_NOALLOC_MAX_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_noalloc_ptr[MAX_DEVICES];   // device address of the array, per device; null until looked up

}  // namespace

GB_EXPORT int gb_sample_noalloc(const float* logits, const float* temperature, const int32_t* top_k,
                                const float* top_p, const float* u, int32_t* out, int R, int V,
                                cudaStream_t stream) {
  if (R <= 0) return GB_OK;
  if (V <= 0) return gb::fail(GB_BAD_ARGUMENT, "cannot sample from empty logits");
  if ((long long)R * V > (long long)GB_SAMPLE_NOALLOC_MAX_FLOATS)
    return gb::fail(GB_BAD_ARGUMENT,
                    "gb_sample_noalloc: %d rows of %d logits need %lld floats of work space, the built-in "
                    "array holds %d; use gb_sample with the caller's own scratch",
                    R, V, (long long)R * V, (int)GB_SAMPLE_NOALLOC_MAX_FLOATS);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "gb_sample_noalloc: %s", cudaGetErrorString(e));
  if (device < 0 || device >= MAX_DEVICES)
    return gb::fail(GB_UNSUPPORTED, "gb_sample_noalloc: device %d is beyond the %d this table holds", device,
                    MAX_DEVICES);
  if (g_noalloc_ptr[device] == nullptr) {
    // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return gb::fail(GB_CUDA_ERROR, "gb_sample_noalloc: cannot find the work space on device %d: %s", device,
                      cudaGetErrorString(e));
    g_noalloc_ptr[device] = p;
  }
  return launch_sample(logits, temperature, top_k, top_p, u, out, g_noalloc_ptr[device], R, V, stream);
}
