// Causal grouped-query attention over the paged cache, one warp per (token,
// query head), 32-bit arithmetic throughout: the attention of the 32-bit path
// and the check beside the tensor-core kernel.
//
// garuda/src/llama/mod.rs:793-818: query head h reads kv head h / g; score
// s_j = dot(q, K_j) * scale with the scale multiplied after the dot; keys j in
// [start, pos], start = max(0, pos + 1 - window) (garuda/src/cache/mod.rs:333-338);
// softmax with the maximum subtracted (garuda/src/simd/mod.rs:132-158); then the
// sum of p_j V_j in key order. Keys are walked 32 at a time from `start`, with
// a running maximum and sum, so the result for a token does not depend on what
// else is in the batch or on how its prompt was cut.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simple_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                        const int32_t* __restrict__ block_table, int table_width,
                        const int32_t* __restrict__ cu_q, const int32_t* __restrict__ kv_lens,
                        const int32_t* __restrict__ token_req, T* __restrict__ out, int Hq, int Hkv, int hd,
                        float scale, int window, int page_size) {
  __shared__ float q_s[WARPS][MAX_HD];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= Hq) return;
  const int r = token_req[t];
  const int q_len = cu_q[r + 1] - cu_q[r];
  const int pos = kv_lens[r] - q_len + (t - cu_q[r]);
  const int start = window > 0 ? max(0, pos + 1 - window) : 0;
  const int kvh = h / (Hq / Hkv);
  const int32_t* table = block_table + (size_t)r * table_width;

  const T* qr = q + ((size_t)t * Hq + h) * hd;
  for (int c = lane; c < hd; c += 32) q_s[warp][c] = gb::to_float<T>(qr[c]);
  __syncwarp();

  const int nacc = (hd + 31) / 32;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = start; base <= pos; base += 32) {
    const int j = base + lane;
    const bool valid = j <= pos;
    long long row = -1;  // row of this lane's key in the pool, in units of hd elements
    if (valid) {
      const int page = table[j / page_size];
      if (page >= 0) row = ((long long)page * Hkv + kvh) * page_size + (j % page_size);
    }
    float s = -INFINITY;
    if (row >= 0) {
      const T* kr = k_pool + row * hd;
      float dot = 0.f;
      for (int c = 0; c < hd; ++c) dot = fmaf(q_s[warp][c], gb::to_float<T>(kr[c]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, gb::warp_max(s));
    const float p = row >= 0 ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + gb::warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
    const int n_here = min(32, pos - base + 1);
    for (int jj = 0; jj < n_here; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long rj = __shfl_sync(0xffffffffu, row, jj);
      if (rj < 0) continue;
      const T* vr = v_pool + rj * hd;
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int c = lane + 32 * i;
        if (i < nacc && c < hd) acc[i] = fmaf(pj, gb::to_float<T>(vr[c]), acc[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* o = out + ((size_t)t * Hq + h) * hd;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int c = lane + 32 * i;
    if (i < nacc && c < hd) o[c] = gb::from_float<T>(acc[i] * inv);
  }
}

}  // namespace

GB_EXPORT int gb_attention_simple(const void* q, const void* k_pool, const void* v_pool, int dtype,
                                  const int32_t* block_table, int table_width, const int32_t* cu_q,
                                  const int32_t* kv_lens, const int32_t* token_req, void* out, int T,
                                  int Hq, int Hkv, int hd, float scale, int window, int page_size,
                                  cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (hd > MAX_HD || hd < 1)
    return gb::fail(GB_UNSUPPORTED, "attention: head_dim %d is outside 1..%d", hd, MAX_HD);
  if (Hkv < 1 || Hq % Hkv) return gb::fail(GB_BAD_ARGUMENT, "attention: %d query heads for %d kv heads", Hq, Hkv);
  dim3 grid(T, (Hq + WARPS - 1) / WARPS);
  return GB_DISPATCH_DTYPE(dtype, TT, [&]() -> int {
    attention_simple_kernel<TT><<<grid, WARPS * 32, 0, stream>>>(
        (const TT*)q, (const TT*)k_pool, (const TT*)v_pool, block_table, table_width, cu_q, kv_lens,
        token_req, (TT*)out, Hq, Hkv, hd, scale, window, page_size);
    return gb::check_launch("attention_simple");
  });
}
