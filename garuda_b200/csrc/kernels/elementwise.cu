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
  gb::pdl_launch_dependents();
  gb::pdl_wait();
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
  gb::pdl_launch_dependents();
  gb::pdl_wait();
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

template <typename OT>
__device__ __forceinline__ void store4(OT* p, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&lo);
  v.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

// Rows of up to 4096 values whose length is a multiple of 4: the row is read once, 16 bytes per
// load, and kept in registers between the sum of squares and the scaling.
template <typename WT, typename OT>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, const WT* __restrict__ w, float eps, OT* __restrict__ out,
                   const int32_t* __restrict__ rows, int d) {
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * d);
  const int nvec = d >> 2;
  float4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + i * 256;
    v[i] = c < nvec ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  __shared__ float warp_part[8];
  __shared__ float scale_s;
  ss = gb::warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_part[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float t = lane < 8 ? warp_part[lane] : 0.f;
    t = gb::warp_sum(t);
    if (lane == 0) scale_s = 1.0f / sqrtf(t / (float)d + eps);
  }
  __syncthreads();
  const float scale = scale_s;
  OT* o = out + (size_t)r * d;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c >= nvec) continue;
    const float w0 = gb::to_float<WT>(w[4 * c]), w1 = gb::to_float<WT>(w[4 * c + 1]);
    const float w2 = gb::to_float<WT>(w[4 * c + 2]), w3 = gb::to_float<WT>(w[4 * c + 3]);
    store4<OT>(o + 4 * c, (v[i].x * scale) * w0, (v[i].y * scale) * w1, (v[i].z * scale) * w2,
               (v[i].w * scale) * w3);
  }
}

// ------------------------------------------------- rotary + cache write
// One block per token. Heads [0, Hq) are queries, [Hq, Hq+Hkv) keys, [Hq+Hkv, Hq+2Hkv) values.
// Angle = (float)pos * inv_freq[i], in 32-bit; sine and cosine are computed once per token and pair.
template <typename IT, typename OT>
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(const IT* __restrict__ qkv, int row_stride, OT* __restrict__ q_out,
                      OT* __restrict__ k_pool, OT* __restrict__ v_pool,
                      const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                      const int32_t* __restrict__ block_table, int table_width, int Hq, int Hkv, int hd,
                      const float* __restrict__ inv_freq, int interleaved, int page_size) {
  __shared__ float sin_s[128], cos_s[128];   // head_dim / 2 <= 128
  gb::pdl_launch_dependents();
  gb::pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = hd >> 1;
  const bool rotate = inv_freq != nullptr;
  if (rotate) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
  }
  long long cache_row = -1;   // row of this token in the pools, in units of one head's page_size * hd block
  if (Hkv > 0) {
    const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    // no page behind this position: the host refuses such a step; nothing is stored
    if (page >= 0) cache_row = (long long)page * Hkv;
  }
  __syncthreads();
  const IT* src = qkv + (size_t)t * row_stride;
  // queries and keys: pairs
  const int rot_heads = Hq + Hkv;
  for (int e = threadIdx.x; e < rot_heads * half; e += blockDim.x) {
    const int head = e / half, i = e % half;
    const int ia = interleaved ? 2 * i : i;
    const int ib = interleaved ? 2 * i + 1 : i + half;
    const IT* s = src + (size_t)head * hd;
    OT* dst;
    if (head < Hq) {
      dst = q_out + ((size_t)t * Hq + head) * hd;
    } else {
      if (cache_row < 0) continue;
      dst = k_pool + ((cache_row + (head - Hq)) * page_size + (pos % page_size)) * hd;
    }
    const float a = gb::to_float<IT>(s[ia]), b = gb::to_float<IT>(s[ib]);
    if (rotate) {
      dst[ia] = gb::from_float<OT>(a * cos_s[i] - b * sin_s[i]);
      dst[ib] = gb::from_float<OT>(a * sin_s[i] + b * cos_s[i]);
    } else {
      dst[ia] = gb::from_float<OT>(a);
      dst[ib] = gb::from_float<OT>(b);
    }
  }
  // values: a copy
  if (cache_row >= 0) {
    const IT* vs = src + (size_t)(Hq + Hkv) * hd;
    for (int e = threadIdx.x; e < Hkv * hd; e += blockDim.x) {
      const int head = e / hd, c = e % hd;
      v_pool[((cache_row + head) * page_size + (pos % page_size)) * hd + c] =
          gb::from_float<OT>(gb::to_float<IT>(vs[e]));
    }
  }
}

// hd: the rotated width (pairs lie within it); head_stride: the distance between heads, which is
// larger than hd when only the first channels of every head are rotated.
__global__ void rope_inplace_kernel(float* __restrict__ x, int row_stride, int head_stride, int H, int hd,
                                    const int32_t* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int interleaved) {
  const int t = blockIdx.x, head = blockIdx.y;
  float* v = x + (size_t)t * row_stride + (size_t)head * head_stride;
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
// gate_up rows hold either [gate(F) | up(F)] (group 0), or gate and up packed in groups of 64:
// columns [128 q, 128 q + 64) gate features 64 q .., the next 64 their up values (group 64).
template <typename IT, typename OT>
__global__ void silu_mul_kernel(const IT* __restrict__ gate_up, OT* __restrict__ out, int M, int F, int group,
                                int row_stride) {
  const size_t n = (size_t)M * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / F, f = i % F;
    const size_t gi = group ? (f / group) * 2 * group + f % group : f;
    const size_t ui = group ? gi + group : F + f;
    const float g = gb::to_float<IT>(gate_up[m * row_stride + gi]);
    const float u = gb::to_float<IT>(gate_up[m * row_stride + ui]);
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
    return gb::check_pdl_launch(gb::launch_pdl(embedding_kernel<TT>, dim3(T), dim3(256), 0, stream, dim3(1, 1, 1),
                                               (const TT*)table, ids, out, d, vocab), "embedding");
  });
}

GB_EXPORT int gb_rmsnorm(const float* x, const void* w, int w_dtype, float eps, void* out, int out_dtype,
                         const int32_t* rows, int n_rows, int d, cudaStream_t stream) {
  if (n_rows <= 0) return GB_OK;
  const int block = d >= 1024 ? 256 : 128;
  return GB_DISPATCH_DTYPE(w_dtype, WT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      if (d % 4 == 0 && d <= 4096 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0)
        return gb::check_pdl_launch(gb::launch_pdl(rmsnorm_vec_kernel<WT, OT>, dim3(n_rows), dim3(256), 0, stream, dim3(1, 1, 1),
                                                   x, (const WT*)w, eps, (OT*)out, rows, d), "rmsnorm");
      return gb::check_pdl_launch(gb::launch_pdl(rmsnorm_kernel<WT, OT>, dim3(n_rows), dim3(block), 0, stream, dim3(1, 1, 1),
                                                 x, (const WT*)w, eps, (OT*)out, rows, d), "rmsnorm");
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
  if (hd > 256) return gb::fail(GB_UNSUPPORTED, "rope_kv_append: head_dim %d is larger than 256", hd);
  const int work = (Hq + Hkv) * (hd / 2);
  const int block = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      return gb::check_pdl_launch(
          gb::launch_pdl(rope_kv_append_kernel<IT, OT>, dim3(T), dim3(block), 0, stream, dim3(1, 1, 1), (const IT*)qkv,
                         row_stride, (OT*)q_out, (OT*)k_pool, (OT*)v_pool, positions, token_req, block_table,
                         table_width, Hq, Hkv, hd, inv_freq, interleaved, page_size),
          "rope_kv_append");
    });
  });
}

// out[t][i] = (cos, sin)((float)positions[t] * inv_freq[i]) for i < half: the rotation's angles
// (garuda/src/simd/mod.rs:196-206) once per step, for every layer's fused epilogue to read.
__global__ void rope_table_kernel(const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ out, int T, int half) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, i = idx % half;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  out[idx] = make_float2(cs, sn);
}

// A plain launch on purpose: kernels after it that start early (programmatic dependent launch) may
// read the table before their dependency wait, which is safe only because this kernel gives no
// early start signal, so that they cannot begin before it has finished.
GB_EXPORT int gb_rope_table(const int32_t* positions, const float* inv_freq, float* out, int T, int half,
                            cudaStream_t stream) {
  if (T <= 0 || half <= 0) return GB_OK;
  const int n = T * half;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(positions, inv_freq, reinterpret_cast<float2*>(out), T, half);
  return gb::check_launch("rope_table");
}

GB_EXPORT int gb_rope_inplace(float* x, int row_stride, int head_stride, int T, int H, int hd,
                              const int32_t* positions, const float* inv_freq, int interleaved,
                              cudaStream_t stream) {
  if (T <= 0 || H <= 0) return GB_OK;
  if (hd % 2) return gb::fail(GB_UNSUPPORTED, "rope_inplace: the rotated width %d is odd", hd);
  if (head_stride < hd) return gb::fail(GB_BAD_ARGUMENT, "rope_inplace: heads %d apart are narrower than %d", head_stride, hd);
  dim3 grid(T, H);
  rope_inplace_kernel<<<grid, 32, 0, stream>>>(x, row_stride, head_stride, H, hd, positions, inv_freq, interleaved);
  return gb::check_launch("rope_inplace");
}

GB_EXPORT int gb_silu_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, int M, int F, int group,
                          int row_stride, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return GB_OK;
  return GB_DISPATCH_DTYPE(in_dtype, IT, [&]() -> int {
    return GB_DISPATCH_DTYPE(out_dtype, OT, [&]() -> int {
      silu_mul_kernel<IT, OT><<<grid_for((size_t)M * F, 256), 256, 0, stream>>>(
          (const IT*)gate_up, (OT*)out, M, F, group, row_stride);
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
