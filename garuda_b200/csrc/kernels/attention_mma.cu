// bfloat16 causal grouped-query attention over the paged cache on the tensor
// cores (mma.sync m16n8k16, 32-bit accumulation), flash-style: keys and values
// are walked in tiles of 64 with a running maximum and sum, so nothing of size
// [queries, keys] is ever stored.
//
// garuda/src/llama/mod.rs:793-818: s_j = dot(q, K_j) * scale over keys
// [start, pos], softmax with the maximum subtracted, sum of p_j V_j; query head h
// reads kv head h / g. start = max(0, pos + 1 - window) with a window
// (garuda/src/cache/mod.rs:333-338). The scale is applied to the 32-bit dot
// product, the softmax is 32-bit; probabilities are rounded to bfloat16 only as
// an operand of the second matrix product.
//
// The rows of a query tile are (token, head-of-the-group) pairs that share one
// kv head of one request, so a K/V tile is read once for the whole group.
// Two variants of one kernel:
//  * TILE: 64 rows per CTA, 16 per warp; every warp walks all key tiles. For
//    prompt portions.
//  * SPLIT: at most 16 rows per CTA (a decode token's group); the four warps
//    share the rows and split each key tile between them, and CTAs split a
//    request's keys between them too. Partial results (unnormalised sum,
//    maximum, denominator) go to scratch memory; the CTA that finishes last
//    (a ticket counter per request and kv head) merges them.
// A request belongs to SPLIT if q_len * g <= 16, else to TILE; each kernel skips
// the other's requests.
//
// Compiled per head size: GB_HEAD_DIM (a multiple of 16, at most 128).
#include "common.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 64
#endif

namespace {

constexpr int HD = GB_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head_dim must be a multiple of 16 up to 128");
constexpr int KT = 64;              // keys per tile
constexpr int PAD = 8;              // bf16 of padding per shared-memory row (16 bytes)
constexpr int LD = HD + PAD;        // shared-memory row length in bf16
constexpr int THREADS = 128;
constexpr int ROWS_TILE = 64;
constexpr int ROWS_SPLIT = 16;
// Key tiles in flight per CTA. A decode CTA has little arithmetic per byte, so what matters is how
// many bytes it has asked for at once: four tiles. A prompt CTA reuses each tile for 64 rows: two.
constexpr int DEPTH_TILE = 2;
constexpr int DEPTH_SPLIT = 4;
constexpr float LOG2E = 1.4426950408889634f;

// Compiled in with -DGB_TIMELINE only: time stamps per CTA of the split kernel.
#ifdef GB_TIMELINE
__device__ unsigned long long g_timeline[8 * 4096];
__device__ __forceinline__ unsigned long long timeline_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define GB_STAMP(i)                                                                                   \
  do {                                                                                                \
    if (SPLIT && threadIdx.x == 0) {                                                                  \
      const int cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);                 \
      if (cta < 4096) g_timeline[8 * cta + (i)] = timeline_now();                                     \
    }                                                                                                 \
  } while (0)
#else
#define GB_STAMP(i) do {} while (0)
#endif

struct Params {
  const __nv_bfloat16* q;        // [T, Hq, HD]
  const __nv_bfloat16* k_pool;   // [pages, Hkv, page_size, HD]
  const __nv_bfloat16* v_pool;
  __nv_bfloat16* out;            // [T, Hq * HD]
  float* partial;                // SPLIT with several splits: [T * Hq, splits, HD + 2]
  int* counters;                 // SPLIT with several splits: [R * Hkv] tickets, zero between launches
  const int32_t* block_table;    // [R, table_width]
  const int32_t* cu_q;           // [R + 1]
  const int32_t* kv_lens;        // [R]
  int table_width, Hq, Hkv, g, window, page_size, num_splits;
  float scale_log2;              // scale * log2(e)
};

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Keys [tile_start, tile_start + KT) of one kv head into shared memory, 16 bytes
// per copy; keys outside [lo, hi] or without a page become zeros. Two threads
// share a key row, so each thread looks one page up per tile.
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const Params& p,
                                             const int32_t* table, int kvh, int tile_start, int lo, int hi) {
  constexpr int CHUNKS = HD / 8;  // 16-byte chunks per row
  static_assert(KT * 2 == THREADS && CHUNKS % 2 == 0, "two threads per key row");
  const int row = threadIdx.x >> 1, first = (threadIdx.x & 1) * (CHUNKS / 2);
  const int j = tile_start + row;
  bool valid = j >= lo && j <= hi;
  size_t off = 0;
  if (valid) {
    const int page = table[j / p.page_size];
    valid = page >= 0;
    if (valid) off = (((size_t)page * p.Hkv + kvh) * p.page_size + (j % p.page_size)) * HD;
  }
#pragma unroll
  for (int c = 0; c < CHUNKS / 2; ++c) {
    const int ch = first + c;
    cp_async_16(ks + row * LD + ch * 8, p.k_pool + off + ch * 8, valid);
    cp_async_16(vs + row * LD + ch * 8, p.v_pool + off + ch * 8, valid);
  }
}

template <bool SPLIT>
__global__ void __launch_bounds__(THREADS)
attention_mma_kernel(const Params p) {
  constexpr int ROWS = SPLIT ? ROWS_SPLIT : ROWS_TILE;
  constexpr int DEPTH = SPLIT ? DEPTH_SPLIT : DEPTH_TILE;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [ROWS][LD]
  __nv_bfloat16* kv = qs + ROWS * LD;                               // DEPTH stages x (K, V) x [KT][LD]

  GB_STAMP(0);
  gb::pdl_launch_dependents();
  // The batch's lengths and block tables were copied in before the step's first kernel: they may be
  // read at once. Queries and this step's own keys and values come from the kernels in front.
  const int r = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  const int rows_total = q_len * p.g;
  const bool small = rows_total <= ROWS_SPLIT;
  if (small != SPLIT || q_len <= 0) return;
  const int kv_len = p.kv_lens[r];
  const int32_t* table = p.block_table + (size_t)r * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // rows of this CTA: row = token_local * g + head_of_group
  const int tokens_per_tile = SPLIT ? q_len : ROWS / p.g;
  const int tok0 = SPLIT ? 0 : blockIdx.x * tokens_per_tile;
  if (tok0 >= q_len) return;
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int nrows = ntok * p.g;
  const int pos0 = kv_len - q_len + tok0;            // position of the tile's first token
  const int pos_last = pos0 + ntok - 1;
  const int lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;   // first key any row reads
  const int hi = pos_last;                                         // last key any row reads

  // key tiles this CTA walks
  const int first_tile = lo / KT;
  int tile_begin = first_tile, tile_end = hi / KT + 1;
  if (SPLIT && p.num_splits > 1) {
    const int total = tile_end - first_tile;
    const int per = (total + p.num_splits - 1) / p.num_splits;
    tile_begin = first_tile + blockIdx.x * per;
    tile_end = min(tile_end, tile_begin + per);
  }

  // Keys and values of earlier steps are final: a decode CTA asks for its tiles of them before
  // waiting for the kernels in front, so that they arrive while those still run. One commit group
  // per tile slot, empty if the slot has no tile or its tile holds positions of this step.
  const int first_new = kv_len - q_len;
  auto is_old = [&](int tile) { return SPLIT && (tile + 1) * KT <= first_new; };
  for (int d = 0; d < DEPTH - 1; ++d) {
    const int tile = tile_begin + d;
    if (tile < tile_end && is_old(tile)) {
      __nv_bfloat16* kd = kv + d * 2 * KT * LD;
      load_kv_tile(kd, kd + KT * LD, p, table, kvh, tile * KT, lo, hi);
    }
    cp_async_commit();
  }
  gb::pdl_wait();
  GB_STAMP(1);

  // ---- queries into shared memory (rows beyond nrows are zeros), and the tiles not asked for yet
  {
    constexpr int CHUNKS = HD / 8;
    for (int c = threadIdx.x; c < ROWS * CHUNKS; c += THREADS) {
      const int row = c / CHUNKS, ch = c % CHUNKS;
      const bool valid = row < nrows;
      const int tok = row / p.g, gh = row % p.g;
      const __nv_bfloat16* src =
          p.q + ((size_t)(q_begin + tok0 + (valid ? tok : 0)) * p.Hq + kvh * p.g + (valid ? gh : 0)) * HD + ch * 8;
      cp_async_16(qs + row * LD + ch * 8, src, valid);
    }
  }
  for (int d = 0; d < DEPTH - 1; ++d) {
    const int tile = tile_begin + d;
    if (tile < tile_end && !is_old(tile)) {
      __nv_bfloat16* kd = kv + d * 2 * KT * LD;
      load_kv_tile(kd, kd + KT * LD, p, table, kvh, tile * KT, lo, hi);
    }
  }
  cp_async_commit();

  // this thread's two rows (lane / 4 and + 8) of the warp's 16
  const int wrow0 = SPLIT ? 0 : warp * 16;
  int row_pos[2], row_start[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = wrow0 + lane / 4 + 8 * i;
    if (row < nrows) {
      row_pos[i] = pos0 + row / p.g;
      row_start[i] = p.window > 0 ? max(0, row_pos[i] + 1 - p.window) : 0;
    } else {
      row_pos[i] = -1;  // no key is valid for a padding row
      row_start[i] = 0;
    }
  }

  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  uint32_t qf[HD / 16][4];
  bool q_loaded = false;

  // keys of a tile that this warp handles: all 64 (TILE) or 16 of them (SPLIT)
  constexpr int NB = SPLIT ? 2 : 8;          // 8-key blocks per warp per tile
  const int key_off = SPLIT ? warp * 16 : 0;

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int stage = (tile - tile_begin) % DEPTH;
    __nv_bfloat16* ks = kv + stage * 2 * KT * LD;
    __nv_bfloat16* vs = ks + KT * LD;
    if (tile + DEPTH - 1 < tile_end) {
      // into the stage that the previous iteration finished with
      __nv_bfloat16* kn = kv + ((tile - tile_begin + DEPTH - 1) % DEPTH) * 2 * KT * LD;
      load_kv_tile(kn, kn + KT * LD, p, table, kvh, (tile + DEPTH - 1) * KT, lo, hi);
    }
    cp_async_commit();
    // Everything but the DEPTH - 1 newest groups has landed: this tile has. Before the first tile
    // the queries' group (the newest but one) must have landed too: wait for all of them.
    if (tile == tile_begin) cp_async_wait<0>();
    else cp_async_wait<DEPTH - 1>();
    __syncthreads();
    if (tile == tile_begin) GB_STAMP(2);

    if (!q_loaded) {
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (wrow0 + (lane % 16)) * LD + kk * 16 + (lane / 16) * 8);
      q_loaded = true;
    }

    // ---- S = Q K^T for this warp's keys
    float s[NB][4];
#pragma unroll
    for (int n = 0; n < NB; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < NB / 2; ++n2) {
        uint32_t b[4];
        const int key = key_off + n2 * 16 + (lane % 8) + (lane / 16) * 8;
        ldmatrix_x4(b, ks + key * LD + kk * 16 + ((lane / 8) % 2) * 8);
        mma_16816(s[2 * n2], qf[kk], b[0], b[1]);
        mma_16816(s[2 * n2 + 1], qf[kk], b[2], b[3]);
      }
    }

    // ---- scale, mask, running softmax (32-bit)
    const int tile_key0 = tile * KT + key_off;
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int n = 0; n < NB; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = tile_key0 + n * 8 + (lane % 4) * 2 + (e & 1);
        const bool ok = j >= row_start[i] && j <= row_pos[i];
        s[n][e] = ok ? s[n][e] * p.scale_log2 : -INFINITY;
        m_new[i] = fmaxf(m_new[i], s[n][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
    }
    float corr[2], m_use[2], l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_use[i] = m_new[i] == -INFINITY ? 0.f : m_new[i];     // nothing valid yet: avoid inf - inf
      corr[i] = m_run[i] == -INFINITY ? 0.f : exp2f(m_run[i] - m_use[i]);
      m_run[i] = m_new[i];
    }
    uint32_t pf[NB / 2][4];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      float pr[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pr[e] = exp2f(s[n][e] - m_use[e >> 1]);   // exp2(-inf) = 0 for masked keys
        l_add[e >> 1] += pr[e];
      }
      pf[n / 2][(n % 2) * 2 + 0] = pack_bf16(pr[0], pr[1]);
      pf[n / 2][(n % 2) * 2 + 1] = pack_bf16(pr[2], pr[3]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_add[i];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < NB / 2; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        uint32_t b[4];
        const int key = key_off + kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
        ldmatrix_x4_trans(b, vs + key * LD + n2 * 16 + (lane / 16) * 8);
        mma_16816(o[2 * n2], pf[kk], b[0], b[1]);
        mma_16816(o[2 * n2 + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // the stage may be overwritten by the next iteration's loads
  }
  cp_async_wait<0>();
  GB_STAMP(3);

  // the denominators: sum over the four threads that share a row
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }

  if (!SPLIT) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = wrow0 + lane / 4 + 8 * i;
      if (row >= nrows) continue;
      const int tok = row / p.g, gh = row % p.g;
      const float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + tok) * p.Hq + kvh * p.g + gh) * HD;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        const uint32_t v = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
        *reinterpret_cast<uint32_t*>(dst + n * 8 + (lane % 4) * 2) = v;
      }
    }
    return;
  }

  // ---- SPLIT: merge the four warps (each saw a quarter of every tile's keys)
  __syncthreads();
  float* red = reinterpret_cast<float*>(kv);            // [4 warps][16 rows][HD + 2]
  constexpr int RS = HD + 2;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = lane / 4 + 8 * i;
    float* dst = red + (warp * 16 + row) * RS;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      dst[n * 8 + (lane % 4) * 2] = o[n][2 * i];
      dst[n * 8 + (lane % 4) * 2 + 1] = o[n][2 * i + 1];
    }
    if (lane % 4 == 0) {
      dst[HD] = m_run[i];
      dst[HD + 1] = l_run[i];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * HD; idx += THREADS) {
    const int row = idx / HD, c = idx % HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, red[(w * 16 + row) * RS + HD]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red[(w * 16 + row) * RS + HD];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
      acc += f * red[(w * 16 + row) * RS + c];
      l += f * red[(w * 16 + row) * RS + HD + 1];
    }
    const int tok = row / p.g, gh = row % p.g;
    const size_t orow = (size_t)(q_begin + tok) * p.Hq + kvh * p.g + gh;
    if (p.num_splits > 1) {
      float* dst = p.partial + (orow * p.num_splits + blockIdx.x) * RS;
      dst[c] = acc;
      if (c == 0) { dst[HD] = m; dst[HD + 1] = l; }
    } else {
      p.out[orow * HD + c] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
  }
  if (p.num_splits == 1) return;
  GB_STAMP(4);

  // ---- the CTA that finishes last for this (request, kv head) merges the splits
  __shared__ int ticket_s;
  __threadfence();
  __syncthreads();
  int* counter = p.counters + (size_t)r * p.Hkv + kvh;
  if (threadIdx.x == 0) ticket_s = atomicAdd(counter, 1);
  __syncthreads();
  GB_STAMP(5);
  if (ticket_s != p.num_splits - 1) return;
  __threadfence();
  const int S = p.num_splits;                           // at most 64
  float* fac = red;                                     // [nrows][S]: weight of each split
  float* inv = red + ROWS_SPLIT * 64;                   // [nrows]: 1 / denominator
  for (int idx = threadIdx.x; idx < nrows * S; idx += THREADS) {
    const int row = idx / S, sp = idx % S;
    const size_t orow = (size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g;
    fac[row * 64 + sp] = __ldcg(p.partial + (orow * S + sp) * RS + HD);      // its maximum, for now
  }
  __syncthreads();
  if (threadIdx.x < nrows) {
    const int row = threadIdx.x;
    const size_t orow = (size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g;
    float m = -INFINITY;
    for (int sp = 0; sp < S; ++sp) m = fmaxf(m, fac[row * 64 + sp]);
    float l = 0.f;
    for (int sp = 0; sp < S; ++sp) {
      const float ms = fac[row * 64 + sp];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - m);
      fac[row * 64 + sp] = f;
      l += f * __ldcg(p.partial + (orow * S + sp) * RS + HD + 1);
    }
    inv[row] = l > 0.f ? 1.0f / l : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * HD; idx += THREADS) {
    const int row = idx / HD, c = idx % HD;
    const size_t orow = (size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g;
    const float* src = p.partial + orow * S * RS + c;
    float acc = 0.f;
    for (int sp = 0; sp < S; ++sp) acc += fac[row * 64 + sp] * __ldcg(src + (size_t)sp * RS);
    p.out[orow * HD + c] = __float2bfloat16_rn(acc * inv[row]);
  }
  if (threadIdx.x == 0) *counter = 0;     // ready for the next launch
  GB_STAMP(6);
}

constexpr int smem_bytes(bool split) {
  return ((split ? ROWS_SPLIT : ROWS_TILE) * LD + (split ? DEPTH_SPLIT : DEPTH_TILE) * 2 * KT * LD) * 2;
}
static_assert(4 * 16 * (HD + 2) * 4 <= 2 * 2 * KT * LD * 2, "merge buffer must fit in the K/V stages");
static_assert((ROWS_SPLIT * 64 + ROWS_SPLIT) * 4 <= 2 * 2 * KT * LD * 2, "split weights must fit in the K/V stages");

}  // namespace

GB_DEFINE_LAST_ERROR()

GB_EXPORT int gb_attention_mma_head_dim() { return HD; }

#ifdef GB_TIMELINE
GB_EXPORT int gb_attention_timeline(unsigned long long* host_out, int ctas) {
  return cudaMemcpyFromSymbol(host_out, g_timeline, sizeof(unsigned long long) * 8 * ctas) == cudaSuccess ? 0 : 1;
}
#endif

// Floats of scratch that gb_attention_mma needs for `num_splits` splits (and R * Hkv ints of
// ticket counters, zero before the first launch; every launch leaves them zero).
GB_EXPORT long long gb_attention_mma_scratch_floats(int T, int Hq, int num_splits) {
  return num_splits > 1 ? (long long)T * Hq * num_splits * (HD + 2) : 0;
}

// q [T, Hq, HD], pools [pages, Hkv, page_size, HD], out [T, Hq*HD], all bfloat16.
// num_splits: CTAs that share the keys of a decode request (1: no scratch needed).
// max_q_len and min_q_len (over the batch's requests) decide which variants are launched.
GB_EXPORT int gb_attention_mma(const void* q, const void* k_pool, const void* v_pool, void* out, float* scratch,
                               int* counters, const int32_t* block_table, int table_width, const int32_t* cu_q,
                               const int32_t* kv_lens, const int32_t* token_req, int T, int R, int Hq, int Hkv,
                               float scale, int window, int page_size, int max_q_len, int min_q_len,
                               int num_splits, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return GB_OK;
  if (Hkv < 1 || Hq % Hkv) return gb::fail(GB_BAD_ARGUMENT, "attention: %d query heads for %d kv heads", Hq, Hkv);
  const int g = Hq / Hkv;
  if (g > ROWS_TILE) return gb::fail(GB_UNSUPPORTED, "attention_mma: a group of %d query heads per kv head", g);
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 64) num_splits = 64;
  if (num_splits > 1 && (!scratch || !counters))
    return gb::fail(GB_BAD_ARGUMENT, "attention_mma: splits need scratch memory and ticket counters");
  Params p;
  p.q = (const __nv_bfloat16*)q; p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  p.out = (__nv_bfloat16*)out; p.partial = scratch; p.counters = counters; p.block_table = block_table; p.cu_q = cu_q;
  p.kv_lens = kv_lens; p.table_width = table_width; p.Hq = Hq; p.Hkv = Hkv; p.g = g; p.window = window;
  p.page_size = page_size; p.num_splits = num_splits; p.scale_log2 = scale * LOG2E;

  static bool configured = false;
  if (!configured) {
    cudaError_t e1 = cudaFuncSetAttribute(attention_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          smem_bytes(false));
    cudaError_t e2 = cudaFuncSetAttribute(attention_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          smem_bytes(true));
    if (e1 != cudaSuccess || e2 != cudaSuccess)
      return gb::fail(GB_CUDA_ERROR, "attention_mma: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    configured = true;
  }
  // SPLIT requests (a decode token's group, or a very short portion), if the batch can hold any
  if (min_q_len * g <= ROWS_SPLIT) {
    int rc = gb::check_pdl_launch(gb::launch_pdl(attention_mma_kernel<true>, dim3(num_splits, Hkv, R), dim3(THREADS),
                                                 smem_bytes(true), stream, 1, p),
                                  "attention_mma (split)");
    if (rc) return rc;
  }
  // TILE requests
  if (max_q_len * g > ROWS_SPLIT) {
    const int tokens_per_tile = ROWS_TILE / g;
    dim3 grid((max_q_len + tokens_per_tile - 1) / tokens_per_tile, Hkv, R);
    return gb::check_pdl_launch(gb::launch_pdl(attention_mma_kernel<false>, grid, dim3(THREADS), smem_bytes(false),
                                               stream, 1, p),
                                "attention_mma (tile)");
  }
  return GB_OK;
}
