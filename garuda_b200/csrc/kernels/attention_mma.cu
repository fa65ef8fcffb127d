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
// Two kernels:
//  * TILE: 64 rows per CTA, 16 per warp; every warp walks all key tiles. For
//    prompt portions.
//  * DECODE: at most 16 rows per CTA (a decode token's group). The CTAs of a
//    thread-block cluster (up to 8) split the request's keys; within a CTA the
//    four tiles of a round are in flight together and each warp takes one. The
//    warps' results are merged in shared memory, the CTAs' results are sent to
//    the cluster's first CTA through distributed shared memory (st.async counted
//    on an mbarrier) and merged there: no scratch in global memory.
// A request belongs to DECODE if q_len * g <= 16, else to TILE; each kernel skips
// the other's requests.
//
// Compiled per head size: GB_HEAD_DIM (a multiple of 16, at most 128).
#include "attention_common.cuh"
#include "error_word.cuh"
#include "attention_mma_core.cuh"
#include "tc_common.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 64
#endif

namespace {

using namespace tc;
using namespace attn_mma;

constexpr int HD = GB_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head_dim must be a multiple of 16 up to 128");
constexpr int PAD = 8;              // bf16 of padding per shared-memory row (16 bytes)
constexpr int LD = HD + PAD;        // shared-memory row length in bf16
constexpr int THREADS = 128;
constexpr int ROWS_TILE = 64;       // query rows per CTA of the TILE kernel
constexpr int ROWS_DECODE = attn::ROWS_DECODE;     // query rows per CTA of the DECODE kernel
constexpr int SLOTS = 4;            // key tiles in flight per DECODE CTA: one per warp and round
constexpr int MAX_CLUSTER = 8;      // CTAs that may share one request's keys
constexpr int RS = HD + 2;          // floats of one row's partial result: sum, then maximum, denominator
constexpr float LOG2E = 1.4426950408889634f;

using attn::Params;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One warp copies NR key rows (keys first_key ..., shared-memory rows first_row ...) of one kv head,
// keys and values, 16 bytes per copy. Consecutive lanes copy consecutive chunks, so that one
// instruction of the warp reads whole 128-byte lines; a row's place in the pool is looked up by
// one lane and handed round with a shuffle. Keys outside [lo, hi] or without a page become zeros.
template <int NR>
__device__ __forceinline__ void warp_load_rows(__nv_bfloat16* ks, __nv_bfloat16* vs, const Params& p,
                                               const int32_t* table, int kvh, int first_key, int first_row,
                                               int lo, int hi) {
  constexpr int CHUNKS = HD / 8;  // 16-byte chunks per row
  constexpr int ITERS = NR * CHUNKS / 32, LOOKUPS = (NR + 31) / 32;
  static_assert(NR * CHUNKS % 32 == 0, "whole warp instructions");
  constexpr uint32_t NONE = 0xFFFFFFFFu;
  const int lane = threadIdx.x & 31;
  uint32_t where[LOOKUPS];        // the row's offset in the pool in units of 16 bytes
#pragma unroll
  for (int h = 0; h < LOOKUPS; ++h) {
    const int j = first_key + lane + 32 * h;
    where[h] = NONE;
    if (lane + 32 * h < NR && j >= lo && j <= hi) {
      const int page = table[j / p.page_size];
      if (page >= 0) where[h] = (uint32_t)((((size_t)page * p.Hkv + kvh) * p.page_size + (j % p.page_size)) * CHUNKS);
    }
  }
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int c = it * 32 + lane, row = c / CHUNKS, ch = c % CHUNKS;
    uint32_t w = __shfl_sync(0xffffffffu, where[0], row & 31);
#pragma unroll
    for (int h = 1; h < LOOKUPS; ++h) {
      const uint32_t other = __shfl_sync(0xffffffffu, where[h], row & 31);
      if (row >> 5 == h) w = other;
    }
    const bool valid = w != NONE;
    const size_t off = valid ? ((size_t)w + ch) * 8 : 0;
    cp_async_16(ks + (first_row + row) * LD + ch * 8, p.k_pool + off, valid);
    cp_async_16(vs + (first_row + row) * LD + ch * 8, p.v_pool + off, valid);
  }
}

// Keys [tile_start, tile_start + KT) of one kv head into shared memory by the whole CTA: each of
// the four warps copies a quarter of the rows.
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const Params& p,
                                             const int32_t* table, int kvh, int tile_start, int lo, int hi) {
  static_assert(KT == 64 && THREADS == 128, "four warps, sixteen rows each");
  const int warp = threadIdx.x >> 5;
  warp_load_rows<16>(ks, vs, p, table, kvh, tile_start + 16 * warp, 16 * warp, lo, hi);
}

// `rows` query rows (row = token_local * g + head_of_group) into shared memory; the rest zeros.
__device__ __forceinline__ void load_queries(__nv_bfloat16* qs, const Params& p, int first_token, int kvh,
                                             int nrows, int rows) {
  constexpr int CHUNKS = HD / 8;
  for (int c = threadIdx.x; c < rows * CHUNKS; c += THREADS) {
    const int row = c / CHUNKS, ch = c % CHUNKS;
    const bool valid = row < nrows;
    const int tok = valid ? row / p.g : 0, gh = valid ? row % p.g : 0;
    cp_async_16(qs + row * LD + ch * 8, p.q + ((size_t)(first_token + tok) * p.Hq + kvh * p.g + gh) * HD + ch * 8,
                valid);
  }
}

// ------------------------------------------------------------------ TILE (prompt portions)
__global__ void __launch_bounds__(THREADS, HD <= 64 ? 4 : 1)
attention_tile_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [ROWS_TILE][LD]
  __nv_bfloat16* kv = qs + ROWS_TILE * LD;                          // 2 stages x (K, V) x [KT][LD]
  gb::pdl_launch_dependents();
  gb::pdl_wait();     // queries and this step's keys and values come from the kernels in front
  const int r = blockIdx.z, kvh = blockIdx.y;
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  if (q_len * p.g <= ROWS_DECODE) return;        // a DECODE request
  const int tokens_per_tile = ROWS_TILE / p.g;
  const int tok0 = blockIdx.x * tokens_per_tile;
  if (tok0 >= q_len) return;
  const int kv_len = p.kv_lens[r];
  const int32_t* table = p.block_table + (size_t)r * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int nrows = ntok * p.g;
  const int pos0 = kv_len - q_len + tok0;            // position of the tile's first token
  const int lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;   // first key any row reads
  const int hi = pos0 + ntok - 1;                                  // last key any row reads
  const int tile_begin = lo / KT, tile_end = hi / KT + 1;

  load_queries(qs, p, q_begin + tok0, kvh, nrows, ROWS_TILE);
  load_kv_tile(kv, kv + KT * LD, p, table, kvh, tile_begin * KT, lo, hi);
  cp_async_commit();

  int row_pos[2], row_start[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = warp * 16 + lane / 4 + 8 * i;
    row_pos[i] = row < nrows ? pos0 + row / p.g : -1;      // no key is valid for a padding row
    row_start[i] = (row < nrows && p.window > 0) ? max(0, row_pos[i] + 1 - p.window) : 0;
  }
  WarpState<HD> st;
  st.reset();
  uint32_t qf[HD / 16][4];
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    __nv_bfloat16* ks = kv + stage * 2 * KT * LD;
    __nv_bfloat16* vs = ks + KT * LD;
    if (tile + 1 < tile_end) {
      __nv_bfloat16* kn = kv + (stage ^ 1) * 2 * KT * LD;
      load_kv_tile(kn, kn + KT * LD, p, table, kvh, (tile + 1) * KT, lo, hi);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (tile == tile_begin) {
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk)
        ldmatrix_x4(qf[kk], qs + (warp * 16 + (lane % 16)) * LD + kk * 16 + (lane / 16) * 8);
    }
    // a tile needs no mask if it lies wholly before the first row's position and inside the last
    // row's window
    const bool full = (tile + 1) * KT - 1 <= pos0 && (p.window <= 0 || tile * KT >= hi + 1 - p.window);
    process_tile<HD>(st, qf, PaddedTile<HD, LD>{ks}, PaddedTile<HD, LD>{vs}, tile * KT, row_pos, row_start, p.scale_log2, full);
    __syncthreads();  // the stage may be overwritten by the next iteration's loads
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
    st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
    const int row = warp * 16 + lane / 4 + 8 * i;
    if (row >= nrows) continue;
    const float inv = st.l[i] > 0.f ? 1.0f / st.l[i] : 0.f;
    __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + row / p.g) * p.Hq + kvh * p.g + row % p.g) * HD;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + (lane % 4) * 2) = pack_bf16(st.o[n][2 * i] * inv, st.o[n][2 * i + 1] * inv);
  }
}

// ------------------------------------------------------------------ DECODE
// grid (ranks, Hkv, R), the `ranks` CTAs along x forming one cluster. Every warp walks its own
// tiles (the CTA's tiles w, w + 4, ...) through a ring of `stages` slots of its own, so that no
// warp waits for another before the merge and the next tile is on its way while one is computed.
__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const Params p, const int stages) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* kv = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [4 warps][stages] x (K, V) x [KT][LD]
  float* red = reinterpret_cast<float*>(kv);                        // after the last tile: [4 warps][16][RS]
  float* mine = red + 4 * ROWS_DECODE * RS;                         // this CTA's merged rows: [16][RS]
  float* parts = reinterpret_cast<float*>(kv + (size_t)stages * 4 * 2 * KT * LD);  // rank 0: [ranks - 1][16][RS]
  __shared__ __align__(8) uint64_t part_bar;

  const int r = blockIdx.z, kvh = blockIdx.y;
  const int rank = blockIdx.x, ranks = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The batch's lengths and block tables were copied in before the step's first kernel: they may be
  // read at once. Queries and this step's own keys and values come from the kernels in front.
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  const int nrows = q_len * p.g;
  if (q_len <= 0 || nrows > ROWS_DECODE) return;   // a TILE request (the whole cluster leaves together)
  const int kv_len = p.kv_lens[r];
  const int32_t* table = p.block_table + (size_t)r * p.table_width;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&part_bar), 1);
    fence_barrier_init();
    if (rank == 0 && ranks > 1)
      mbar_arrive_expect_tx(smem_u32(&part_bar), (uint32_t)(ranks - 1) * nrows * RS * 4);
  }
  __syncthreads();
  if (ranks > 1) cluster_arrive_wait();      // rank 0's barrier is armed before anyone sends to it
  gb::pdl_launch_dependents();

  const int pos0 = kv_len - q_len;                                  // position of the first token
  const int lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;    // first key any row reads
  const int hi = kv_len - 1;
  const int first_tile = lo / KT, total = hi / KT + 1 - first_tile;
  const int per = (total + ranks - 1) / ranks;
  const int tile_begin = first_tile + rank * per;
  const int tile_end = min(hi / KT + 1, tile_begin + per);
  const int mine_n = tile_begin + warp < tile_end ? (tile_end - tile_begin - warp + 3) / 4 : 0;   // this warp's tiles

  int row_pos[2], row_start[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = lane / 4 + 8 * i;
    row_pos[i] = row < nrows ? pos0 + row / p.g : -1;
    row_start[i] = (row < nrows && p.window > 0) ? max(0, row_pos[i] + 1 - p.window) : 0;
  }
  __nv_bfloat16* ring = kv + (size_t)warp * stages * 2 * KT * LD;
  auto issue = [&](int i) {    // the warp's i-th tile into its slot; one group per call, even when empty
    if (i < mine_n) {
      __nv_bfloat16* kd = ring + (size_t)(i % stages) * 2 * KT * LD;
      warp_load_rows<KT>(kd, kd + KT * LD, p, table, kvh, (tile_begin + warp + 4 * i) * KT, 0, lo, hi);
    }
    cp_async_commit();
  };
  // Keys and values of earlier steps are final: tiles that lie wholly before the first token are
  // asked for before waiting for the kernels in front, so that they arrive while those still run.
  // Only a warp's last tile can hold new keys, so the order of the groups stays the tiles' order.
  int issued = 0;
  while (issued < stages && issued < mine_n && (tile_begin + warp + 4 * issued + 1) * KT <= pos0) issue(issued++);
  gb::pdl_wait();
  while (issued < stages) issue(issued++);

  // the query fragments of the m16n8k16 A operand, straight from global memory
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int row = lane / 4 + 8 * (e & 1);
    const __nv_bfloat16* src =
        p.q + ((size_t)(q_begin + (row < nrows ? row / p.g : 0)) * p.Hq + kvh * p.g + (row < nrows ? row % p.g : 0)) * HD +
        (lane % 4) * 2 + 8 * (e >> 1);
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk)
      qf[kk][e] = row < nrows ? *reinterpret_cast<const uint32_t*>(src + kk * 16) : 0u;
  }

  WarpState<HD> st;
  st.reset();
  for (int i = 0; i < mine_n; ++i) {
    if (stages == 1) cp_async_wait<0>(); else cp_async_wait<1>();
    __syncwarp();
    const __nv_bfloat16* ks = ring + (size_t)(i % stages) * 2 * KT * LD;
    process_tile<HD>(st, qf, PaddedTile<HD, LD>{ks}, PaddedTile<HD, LD>{ks + KT * LD}, (tile_begin + warp + 4 * i) * KT, row_pos, row_start, p.scale_log2, false);
    __syncwarp();             // every lane is done with the slot before it is filled again
    issue(i + stages);
  }
  cp_async_wait<0>();
  __syncthreads();            // the slots become the merge buffers
  // ---- the four warps' results into shared memory: [warp][row][RS]
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
    st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
    const int row = lane / 4 + 8 * i;
    if (row >= nrows) continue;
    float* dst = red + (warp * ROWS_DECODE + row) * RS;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
      *reinterpret_cast<float2*>(dst + n * 8 + (lane % 4) * 2) = make_float2(st.o[n][2 * i], st.o[n][2 * i + 1]);
    if (lane % 4 == 0) {
      dst[HD] = st.m[i] * p.scale_log2;     // in units of the exponent, as the merges want it
      dst[HD + 1] = st.l[i];
    }
  }
  __syncthreads();
  // ---- merge the warps: sixteen threads share a row, each computes the row's four weights
  // exp2(m_w - m) itself. A CTA that is alone or leads keeps the result, the others pass it on.
  const bool send = ranks > 1 && rank != 0;
  const uint32_t remote = send ? map_to_rank(smem_u32(parts) + (uint32_t)(rank - 1) * nrows * RS * 4, 0) : 0;
  const uint32_t remote_bar = send ? map_to_rank(smem_u32(&part_bar), 0) : 0;
  const int sub = threadIdx.x & 15;
  for (int row = threadIdx.x >> 4; row < nrows; row += THREADS / 16) {
    float f[4], m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, red[(w * ROWS_DECODE + row) * RS + HD]);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red[(w * ROWS_DECODE + row) * RS + HD];
      f[w] = mw == -INFINITY ? 0.f : fast_exp2(mw - m);
    }
    // columns sub, sub + 16, ...; column HD is the maximum, HD + 1 the denominator (weighted like the sums)
    for (int c = sub; c < RS; c += 16) {
      float v = m;
      if (c != HD) {
        v = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) v += f[w] * red[(w * ROWS_DECODE + row) * RS + c];
      }
      if (send) st_async_f32(remote + (uint32_t)(row * RS + c) * 4, remote_bar, v);
      else mine[row * RS + c] = v;
    }
  }
  if (rank != 0) return;
  if (ranks > 1 && !mbar_wait(smem_u32(&part_bar), 0)) {
    if (threadIdx.x == 0) gb_err::report(5);
    return;
  }
  __syncthreads();
  // ---- rank 0: its own rows and the others' [rank - 1][nrows][RS], in rank order
  for (int row = threadIdx.x >> 4; row < nrows; row += THREADS / 16) {
    float f[MAX_CLUSTER], m = mine[row * RS + HD];
    for (int q = 1; q < ranks; ++q) m = fmaxf(m, parts[((q - 1) * nrows + row) * RS + HD]);
    float l = 0.f;
#pragma unroll
    for (int q = 0; q < MAX_CLUSTER; ++q) {
      f[q] = 0.f;
      if (q < ranks) {
        const float* src = q == 0 ? mine + row * RS : parts + ((q - 1) * nrows + row) * RS;
        f[q] = src[HD] == -INFINITY ? 0.f : fast_exp2(src[HD] - m);
        l += f[q] * src[HD + 1];
      }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    __nv_bfloat16* dst = p.out + ((size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g) * HD;
    for (int c = sub; c < HD; c += 16) {
      float acc = f[0] * mine[row * RS + c];
#pragma unroll
      for (int q = 1; q < MAX_CLUSTER; ++q)
        if (q < ranks) acc += f[q] * parts[((q - 1) * nrows + row) * RS + c];
      dst[c] = __float2bfloat16_rn(acc * inv);
    }
  }
}

constexpr int SMEM_TILE = (ROWS_TILE * LD + 2 * 2 * KT * LD) * 2;
constexpr int smem_decode(int ranks, int stages) {
  return stages * 4 * 2 * KT * LD * 2 + (ranks > 1 ? (ranks - 1) * ROWS_DECODE * RS * 4 : 0);
}
constexpr int MAX_STAGES = smem_decode(MAX_CLUSTER, 2) <= 200 * 1024 ? 2 : 1;
static_assert((4 * ROWS_DECODE + ROWS_DECODE) * RS * 4 <= 4 * 2 * KT * LD * 2, "the merge buffers must fit in the key slots");

}  // namespace

GB_DEFINE_LAST_ERROR()

GB_EXPORT int gb_attention_mma_head_dim() { return HD; }

// Scratch that gb_attention_mma wants for `splits` CTAs per decode request (0: none).
GB_EXPORT long long gb_attention_scratch_bytes(int R, int kv_heads, int splits) {
  return attn::decode_tma_scratch_bytes(R, kv_heads, splits);
}

// How often prompt portions went to the tcgen05 kernel, and decode requests to the kernel that copies
// pages by TMA (for tests and launch counts).
static long long g_tc_tile_launches = 0, g_decode_tma_launches = 0;
GB_EXPORT long long gb_attention_tc_tile_launches() { return g_tc_tile_launches; }
GB_EXPORT long long gb_attention_decode_tma_launches() { return g_decode_tma_launches; }

// Non-zero if a decode CTA gave up waiting for its cluster since the last call; clears it.
GB_EXPORT int gb_attention_error_check() {
  const int tc = attn::tile_tc_error_check();
  const int tma = attn::decode_tma_error_check();
  const int own = gb_err::fetch_and_clear();
  return tc != 0 ? tc : (tma != 0 ? tma : own);
}

// A word of pinned host memory that a kernel's failed wait also writes its code to (null: none).
GB_EXPORT int gb_attention_set_error_sink(int* host_word) {
  const int a = gb_err::set_sink(host_word), b = attn::tile_tc_set_error_sink(host_word);
  const int c = attn::decode_tma_set_error_sink(host_word);
  return a != 0 ? a : (b != 0 ? b : c);
}

// q [T, Hq, HD], pools [pages, Hkv, page_size, HD], out [T, Hq*HD], all bfloat16.
// num_splits: CTAs (one cluster, at most 8) that share the keys of a decode request. stages: slots
// per warp of the decode kernel (2: the next tile is fetched while one is computed; clamped to what
// shared memory holds for this head size).
// max_q_len and min_q_len (over the batch's requests) decide which kernels are launched; num_pages:
// pages in each pool. cluster_merge: for the decode kernel that copies by TMA, whether the CTAs that share
// a request are a thread-block cluster (no scratch) or independent. scratch: work space for the decode kernel that copies by TMA when several CTAs
// share a request (gb_attention_scratch_bytes of it; its first 64 KB zero before the first call, and
// the same memory from call to call, or zeroed again); may be null.
GB_EXPORT int gb_attention_mma(const void* q, const void* k_pool, const void* v_pool, void* out,
                               const int32_t* block_table, int table_width, const int32_t* cu_q,
                               const int32_t* kv_lens, int T, int R, int Hq, int Hkv, float scale, int window,
                               int page_size, int max_q_len, int min_q_len, int num_splits, int stages,
                               long long num_pages, int cluster_merge, void* scratch, long long scratch_bytes,
                               cudaStream_t stream) {
  if (T <= 0 || R <= 0) return GB_OK;
  if (Hkv < 1 || Hq % Hkv) return gb::fail(GB_BAD_ARGUMENT, "attention: %d query heads for %d kv heads", Hq, Hkv);
  const int g = Hq / Hkv;
  if (g > ROWS_TILE) return gb::fail(GB_UNSUPPORTED, "attention_mma: a group of %d query heads per kv head", g);
  // the running maximum is taken before the scale is applied, which needs the scale to be positive
  if (!(scale > 0.f)) return gb::fail(GB_UNSUPPORTED, "attention_mma: scale %g is not positive", (double)scale);
  const int tma_splits = num_splits;
  num_splits = num_splits < 1 ? 1 : (num_splits > MAX_CLUSTER ? MAX_CLUSTER : num_splits);
  Params p;
  p.q = (const __nv_bfloat16*)q; p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.table_width = table_width; p.Hq = Hq; p.Hkv = Hkv; p.g = g; p.window = window; p.page_size = page_size;
  p.scale_log2 = scale * LOG2E;

  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e1 = cudaFuncSetAttribute(attention_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TILE);
    cudaError_t e2 = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          smem_decode(MAX_CLUSTER, MAX_STAGES));
    if (e1 != cudaSuccess || e2 != cudaSuccess)
      return gb::fail(GB_CUDA_ERROR, "attention_mma: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    configured.done();
  }
  // DECODE requests (a decode token's group, or a very short portion), if the batch can hold any
  if (min_q_len * g <= ROWS_DECODE && attn::decode_tma_takes(p, num_pages)) {
    int rc = attn::launch_decode_tma(p, num_pages, R, tma_splits, cluster_merge != 0, scratch, scratch_bytes, stream);
    if (rc) return rc;
    ++g_decode_tma_launches;
  } else if (min_q_len * g <= ROWS_DECODE) {
    stages = stages < 1 ? 1 : (stages > MAX_STAGES ? MAX_STAGES : stages);
    int rc = gb::check_pdl_launch(gb::launch_pdl(attention_decode_kernel, dim3(num_splits, Hkv, R), dim3(THREADS),
                                                 smem_decode(num_splits, stages), stream, dim3(num_splits, 1, 1), p,
                                                 stages),
                                  "attention_mma (decode)");
    if (rc) return rc;
  }
  // TILE requests: on the tcgen05 kernel where it takes the shape
  if (max_q_len * g > ROWS_DECODE) {
    if (attn::tile_tc_takes(p, T, num_pages)) {
      ++g_tc_tile_launches;
      return attn::launch_tile_tc(p, T, num_pages, R, max_q_len, stream);
    }
    const int tokens_per_tile = ROWS_TILE / g;
    dim3 grid((max_q_len + tokens_per_tile - 1) / tokens_per_tile, Hkv, R);
    return gb::check_pdl_launch(gb::launch_pdl(attention_tile_kernel, grid, dim3(THREADS), SMEM_TILE, stream, dim3(1, 1, 1), p),
                                "attention_mma (tile)");
  }
  return GB_OK;
}
