// Embedding, RMS norm, rotary positions with the write into the paged cache,
// SiLU-gate and the residual add. All arithmetic is 32-bit; only what is stored
// may be bfloat16. Formulas: garuda/src/simd/mod.rs (rmsnorm :166-173, rope
// :196-206, silu :161-163, add_assign :176-179) and garuda/src/llama/mod.rs
// (embedding row copy :198-200, :1078-1085; norm weight multiply :733-738;
// rotate then store :784-791).
#include "common.cuh"

GB_DEFINE_LAST_ERROR()

namespace {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                 float* __restrict__ out, int d, int vocab) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * d;
  if (id < 0 || id >= vocab) {  // refused on the host before any launch; never read out of range
    for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = gb::to_float<T>(row[c]);
}

// ------------------------------------------------------------------ rmsnorm
// One block per row. sum of squares in 32-bit: per-thread partial sums over a
// strided walk, then a fixed-order tree, so a row's result does not depend on
// which other rows are in the batch.
template <typename WT, typename OT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const WT* __restrict__ w, float eps,
                               OT* __restrict__ out, const int32_t* __restrict__ rows, int d) {
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + (size_t)src * d;
  OT* o = out + (size_t)r * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float v = xr[c];
    ss = fmaf(v, v, ss);
  }
  __shared__ float warp_part[32];
  __shared__ float scale_s;
  ss = gb::warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (blockDim.x >> 5) ? warp_part[lane] : 0.f;
    v = gb::warp_sum(v);
    if (lane == 0) scale_s = 1.0f / sqrtf(v / (float)d + eps);
  }
  __syncthreads();
  const float scale = scale_s;
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    o[c] = gb::from_float<OT>((xr[c] * scale) * gb::to_float<WT>(w[c]));
}

// ------------------------------------------------- rotary + cache write
// One block per (token, head). Heads [0, Hq) are queries, [Hq, Hq+Hkv) keys,
// [Hq+Hkv, Hq+2Hkv) values. Angle = (float)pos * inv_freq[i], in 32-bit.
template <typename IT, typename OT>
__global__ void rope_kv_append_kernel(const IT* __restrict__ qkv, int row_stride, OT* __restrict__ q_out,
                                      OT* __restrict__ k_pool, OT* __restrict__ v_pool,
                                      const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ token_req,
                                      const int32_t* __restrict__ block_table, int table_width,
                                      int Hq, int Hkv, int hd, const float* __restrict__ inv_freq,
                                      int interleaved, int page_size) {
  const int t = blockIdx.x, head = blockIdx.y;
  const int pos = positions[t];
  const IT* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
  OT* dst;
  bool rotate = inv_freq != nullptr;
  if (head < Hq) {
    dst = q_out + ((size_t)t * Hq + head) * hd;
  } else {
    const int kvh = (head - Hq) % Hkv;
    const bool is_v = head >= Hq + Hkv;
    const int req = token_req[t];
    const int page = block_table[(size_t)req * table_width + pos / page_size];
    if (page < 0) return;  // no page behind this position: the host refuses such a step
    OT* pool = is_v ? v_pool : k_pool;
    dst = pool + (((size_t)page * Hkv + kvh) * page_size + (pos % page_size)) * hd;
    if (is_v) rotate = false;
  }
  if (!rotate) {
    for (int c = threadIdx.x; c < hd; c += blockDim.x) dst[c] = gb::from_float<OT>(gb::to_float<IT>(src[c]));
    return;
  }
  const int half = hd >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float ang = (float)pos * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    const int ia = interleaved ? 2 * i : i;
    const int ib = interleaved ? 2 * i + 1 : i + half;
    const float a = gb::to_float<IT>(src[ia]), b = gb::to_float<IT>(src[ib]);
    dst[ia] = gb::from_float<OT>(a * c - b * s);
    dst[ib] = gb::from_float<OT>(a * s + b * c);
  }
}

__global__ void rope_inplace_kernel(float* __restrict__ x, int row_stride, int H, int hd,
                                    const int32_t* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int interleaved) {
  const int t = blockIdx.x, head = blockIdx.y;
  float* v = x + (size_t)t * row_stride + (size_t)head * hd;
  const int pos = positions[t];
  const int half = hd >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float ang = (float)pos * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    const int ia = interleaved ? 2 * i : i;
    const int ib = interleaved ? 2 * i + 1 : i + half;
    const float a = v[ia], b = v[ib];
    v[ia] = a * c - b * s;
    v[ib] = a * s + b * c;
  }
}

// ------------------------------------------------------------ SiLU-gate
template <typename IT, typename OT>
__global__ void silu_mul_kernel(const IT* __restrict__ gate_up, OT* __restrict__ out, int M, int F) {
  const size_t n = (size_t)M * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / F, f = i % F;
    const float g = gb::to_float<IT>(gate_up[m * 2 * F + f]);
    const float u = gb::to_float<IT>(gate_up[m * 2 * F + F + f]);
    out[i] = gb::from_float<OT>((g / (1.0f + expf(-g))) * u);
  }
}

template <typename YT>
__global__ void residual_add_kernel(float* __restrict__ x, const YT* __restrict__ y, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] += gb::to_float<YT>(y[i]);
}

int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  return (int)(g > 148 * 16 ? 148 * 16 : (g ? g : 1));
}

}  // namespace

GB_EXPORT int gb_embedding(const void* table, int table_dtype, const int32_t* ids, float* out, int T,
                           int d, int vocab, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(table_dtype, TT, [&]() -> int {
    embedding_kernel<TT><<<T, 256, 0, stream>>>((const TT*)table, ids, out, d, vocab);
    return gb::check_launch("embedding");
  });
}

GB_EXPORT int gb_rmsnorm(const float* x, const void* w, int w_dtype, float eps, void* out, int out_dtype,
                         const int32_t* rows, int n_rows, int d, cudaStream_t stream) {
  if (n_rows <= 0) return GB_OK;
  const int block = d >= 1024 ? 256 : 128;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      rmsnorm_kernel<WT, OT><<<n_rows, block, 0, stream>>>(x, (const WT*)w, eps, (OT*)out, rows, d);
      return gb::check_launch("rmsnorm");
    });
  });
}

GB_EXPORT int gb_rope_kv_append(const void* qkv, int in_dtype, int row_stride, void* q_out, void* k_pool,
                                void* v_pool, int out_dtype, const int32_t* positions,
                                const int32_t* token_req, const int32_t* block_table, int table_width,
                                int T, int Hq, int Hkv, int hd, const float* inv_freq, int interleaved,
                                int page_size, cudaStream_t stream) {
  if (T <= 0) return GB_OK;
  if (hd % 2) return gb::fail(GB_UNSUPPORTED, "rope_kv_append: head_dim %d is odd", hd);
  if (Hkv > 0 && (!k_pool || !v_pool || !block_table || page_size < 1))
    return gb::fail(GB_BAD_ARGUMENT, "rope_kv_append: kv heads given without a cache to store them in");
  dim3 grid(T, Hq + 2 * Hkv);
  const int block = hd / 2 >= 64 ? 64 : 32;
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      rope_kv_append_kernel<IT, OT><<<grid, block, 0, stream>>>(
          (const IT*)qkv, row_stride, (OT*)q_out, (OT*)k_pool, (OT*)v_pool, positions, token_req,
          block_table, table_width, Hq, Hkv > 0 ? Hkv : 1, hd, inv_freq, interleaved, page_size);
      return gb::check_launch("rope_kv_append");
    });
  });
}

GB_EXPORT int gb_rope_inplace(float* x, int row_stride, int T, int H, int hd, const int32_t* positions,
                              const float* inv_freq, int interleaved, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return GB_OK;
  if (hd % 2) return gb::fail(GB_UNSUPPORTED, "rope_inplace: head_dim %d is odd", hd);
  dim3 grid(T, H);
  rope_inplace_kernel<<<grid, 32, 0, stream>>>(x, row_stride, H, hd, positions, inv_freq, interleaved);
  return gb::check_launch("rope_inplace");
}

GB_EXPORT int gb_silu_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, int M, int F,
                          cudaStream_t stream) {
  if (M <= 0 || F <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      silu_mul_kernel<IT, OT><<<grid_for((size_t)M * F, 256), 256, 0, stream>>>(
          (const IT*)gate_up, (OT*)out, M, F);
      return gb::check_launch("silu_mul");
    });
  });
}

GB_EXPORT int gb_residual_add(float* x, const void* y, int y_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(y_dtype, YT, [&]() -> int {
    residual_add_kernel<YT><<<grid_for((size_t)n, 256), 256, 0, stream>>>(x, (const YT*)y, (size_t)n);
    return gb::check_launch("residual_add");
  });
}
