// Decode attention over the paged cache with the keys and values brought in by TMA.
//
// The same arithmetic as the DECODE kernel of attention_mma.cu (garuda/src/llama/mod.rs:793-818:
// s_j = dot(q, K_j) * scale over keys [start, pos], softmax with the maximum subtracted, sum of
// p_j V_j; query head h reads kv head h / g; a window starts at pos + 1 - window,
// garuda/src/cache/mod.rs:333-338), for requests of at most 16 (token, head-of-group) rows: flash-style
// over tiles of 32 keys on mma.sync m16n8k16 with 32-bit accumulation and a 32-bit softmax. With
// at most 16 query rows the products are a few per cent of what the tensor cores can do and the kernel
// is bound by the stream of keys and values; a tcgen05 product (128 rows) would be seven eighths padding.
//
// What differs is how the cache reaches shared memory. A page of one kv head is one box of a
// four-dimensional tensor map over the pool [pages][kv heads][page_size][head_dim] (two boxes for a
// head of 128: one per 64 channels), written with the 128-byte swizzle that ldmatrix then undoes. One
// lane of a warp issues the copies, two or four per tile of 32 keys, with the pages looked up in the
// block table 32 tiles at a time. The CTA's warps take the tiles in turn (tile i goes to warp i mod W)
// and each warp has a ring of three stages of its own with an mbarrier per stage: it asks for a tile
// three tiles ahead as soon as it is done with the stage that tile goes to, so no warp waits for
// another, and it only ever waits on barriers whose earlier phases it has itself seen complete, which
// is what waiting by phase parity needs. No thread computes an address per 16 bytes, and the CTA needs
// under 100 KB of shared memory, so two fit on an SM. Keys and values of earlier steps are final: their tiles are
// asked for before the wait for the kernels in front (programmatic dependent launch); only the tile
// that holds this step's own keys waits.
//
// Several CTAs (grid x) may split a request's keys, in one of two ways. As a thread-block cluster
// (at most 8, or 4 for heads of 128): their partial results (sums, maximum, denominator per row) go to
// the cluster's first CTA through distributed shared memory (st.async counted on an mbarrier) and are
// merged there in rank order. That is the shortest way (a few requests at 2,048 keys: 7 us against 10),
// but a cluster's CTAs are placed together, which takes longer the more CTAs there are, and the partial
// results take shared memory, so only one CTA fits on an SM. Or independently (up to 16): each CTA
// writes its partial result to scratch memory that the caller provides, publishes it with a fence and
// counts itself on a counter in that scratch; the CTA that counts the last arrival reads all of them
// back and merges them in rank order: the same sum whichever CTA is last. It leaves the counter at zero,
// which is what the next launch expects (the caller zeroes the counters once). That is the way for
// many requests or long contexts (8 requests of 8,192 keys and heads of 128: 46 us against 87).
//
// A page that was given back (block table -1) is a box at page coordinate -1: outside the tensor, it
// reads as zeros. Rows of a page beyond the request's length hold what an earlier owner of the page
// left: their scores are masked, and their value rows are cleared in shared memory before the second
// product (a stray NaN times a zero probability would spoil a sum).
//
// Built for head sizes 64 and 128 and pages of 8 to 128 keys (a power of two); the kernel of
// attention_mma.cu takes everything else. Every wait is bounded.
#include "attention_common.cuh"
#include "attention_mma_core.cuh"
#include "error_word.cuh"
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 64
#endif

#if GB_HEAD_DIM == 64 || GB_HEAD_DIM == 128

namespace {

using namespace tc;
using namespace attn_mma;
using attn::Params;

constexpr int HD = GB_HEAD_DIM;
constexpr int TK = 32;                          // keys per tile
constexpr int HALVES = HD / 64;                 // 64-channel halves of a head: one swizzled 128-byte row each
constexpr int HALF_BYTES = TK * 128;            // [32 keys][128 bytes]
constexpr int OPERAND_BYTES = HALVES * HALF_BYTES;      // a tile's keys (or values)
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;          // 8 KB or 16 KB
constexpr int CONSUMERS = HD == 64 ? 4 : 2;     // warps that compute
constexpr int DEPTH = 3;                        // stages of each warp's own ring
constexpr int STAGES = CONSUMERS * DEPTH;               // 96 KB of rings
constexpr int RING_BYTES = STAGES * STAGE_BYTES;
constexpr int CTHREADS = 32 * CONSUMERS;
constexpr int THREADS = CTHREADS;
constexpr int ROWS = attn::ROWS_DECODE;
constexpr int RS = HD + 2;                      // floats of one row's partial result: sums, maximum, denominator
constexpr int MAX_RANKS = 16;                   // CTAs that may share one request's keys
constexpr int CLUSTER_RANKS = HD == 64 ? 8 : 4; // as a thread-block cluster (their partial results take shared memory)
constexpr unsigned long long DRAIN_LIMIT_NS = 20000000ull;      // waits after a failure: 20 ms

static_assert((CONSUMERS * ROWS + ROWS) * RS * 4 <= RING_BYTES, "the merge buffers must fit in the ring");

constexpr int SMEM_BYTES = 1024 + RING_BYTES;
constexpr int smem_cluster(int ranks) { return SMEM_BYTES + (ranks > 1 ? (ranks - 1) * ROWS * RS * 4 : 0); }
constexpr long long COUNTER_BYTES = 64 * 1024;  // of the caller's scratch: one counter per (request, kv head)

// CLUSTER: the CTAs along x are a thread-block cluster and merge through distributed shared memory.
template <bool CLUSTER>
__global__ void __launch_bounds__(THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            const Params p, const int box_rows, float* __restrict__ partials,
                            int* __restrict__ counters) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t part_bar;
  __shared__ int abort_s;

  const int r = blockIdx.z, kvh = blockIdx.y;
  const int rank = blockIdx.x, ranks = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The batch's lengths and block tables were copied in before the step's first kernel: they may be
  // read at once. Queries and this step's own keys and values come from the kernels in front.
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  const int nrows = q_len * p.g;
  if (q_len <= 0 || nrows > ROWS) return;        // not a decode request
  const int kv_len = p.kv_lens[r];
  const int32_t* table = p.block_table + (size_t)r * p.table_width;

  uint8_t* ring = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
  float* red = reinterpret_cast<float*>(ring);                 // after the last tile: [warps][16][RS]
  float* mine = red + CONSUMERS * ROWS * RS;                    // CLUSTER: this CTA's merged rows [16][RS]
  float* parts = reinterpret_cast<float*>(ring + RING_BYTES);   // CLUSTER, rank 0: [ranks - 1][nrows][RS]

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
    }
    mbar_init(smem_u32(&part_bar), 1);
    abort_s = 0;
    fence_barrier_init();
    if (CLUSTER && rank == 0 && ranks > 1)
      mbar_arrive_expect_tx(smem_u32(&part_bar), (uint32_t)(ranks - 1) * nrows * RS * 4);
    fence_proxy_async();
    prefetch_tensormap(&k_map);
    prefetch_tensormap(&v_map);
  }
  __syncthreads();
  if (CLUSTER && ranks > 1) cluster_arrive_wait();      // rank 0's barrier is armed before anyone sends to it
  gb::pdl_launch_dependents();

  const int pos0 = kv_len - q_len;                                  // position of the first token
  const int lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;    // first key any row reads
  const int hi = kv_len - 1;
  const int first_tile = lo / TK, total = hi / TK + 1 - first_tile;
  const int per = (total + ranks - 1) / ranks;
  const int tile_begin = first_tile + rank * per;
  const int tile_end = min(hi / TK + 1, tile_begin + per);
  const int n_tiles = max(tile_end - tile_begin, 0);
  volatile int* aborted = &abort_s;

  {
    // Every warp walks its own tiles (the CTA's tiles warp, warp + W, ...) through its own ring: lane 0
    // asks for a tile DEPTH tiles ahead as soon as the warp is done with the stage it goes to, so no
    // warp ever waits for another. The pages of 32 tiles are looked up at a time, a tile per lane (one
    // round trip to the block table instead of one per tile), and handed to lane 0 by shuffles.
    const int boxes = TK / box_rows;           // page boxes per tile (box_rows = min(page_size, 32)): 1, 2 or 4
    const int mine_n = warp < n_tiles ? (n_tiles - warp + CONSUMERS - 1) / CONSUMERS : 0;     // this warp's tiles
    int pages[4] = {-1, -1, -1, -1};           // of the warp's tile `looked_up + lane`
    int looked_up = -32;
    bool waited = false;
    auto issue = [&](int t) {                  // the warp's t-th tile into stage t % DEPTH of its ring
      if (t >= mine_n) return;
      if (t >= looked_up + 32) {
        looked_up = t;
        const int key0 = (tile_begin + warp + CONSUMERS * (t + lane)) * TK;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          // beyond the table (a tile's tail past the context) and given-back pages: coordinate -1, zeros
          const int slot = (key0 + b * box_rows) / p.page_size;
          pages[b] = (t + lane < mine_n && b < boxes && slot < p.table_width) ? table[slot] : -1;
        }
      }
      int pg[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) pg[b] = __shfl_sync(0xffffffffu, pages[b], t - looked_up);
      const int key0 = (tile_begin + warp + CONSUMERS * t) * TK;
      // a tile that may hold this step's keys waits for the kernel that writes them
      if (!waited && key0 + TK > pos0) {
        gb::pdl_wait();
        waited = true;
      }
      if (lane == 0) {
        const int s = warp * DEPTH + t % DEPTH;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t kdst = smem_u32(ring + s * STAGE_BYTES), vdst = kdst + OPERAND_BYTES;
        // what the warp read from or wrote to this stage is ordered before the copies that overwrite it
        fence_proxy_async();
        mbar_arrive_expect_tx(bar, STAGE_BYTES);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          if (b >= boxes) break;
          const int row = (key0 + b * box_rows) % p.page_size;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            const uint32_t off = h * HALF_BYTES + b * box_rows * 128;
            tma_load_4d(kdst + off, &k_map, bar, h * 64, row, kvh, pg[b]);
            tma_load_4d(vdst + off, &v_map, bar, h * 64, row, kvh, pg[b]);
          }
        }
      }
    };
    // tiles of earlier steps are asked for before the wait for the kernels in front
    int issued = 0;
    while (issued < DEPTH && issued < mine_n && (tile_begin + warp + CONSUMERS * issued + 1) * TK <= pos0) issue(issued++);
    if (!waited) {
      gb::pdl_wait();            // the queries come from the kernel in front
      waited = true;
    }
    while (issued < DEPTH && issued < mine_n) issue(issued++);

    int row_pos[2], row_start[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = lane / 4 + 8 * i;
      row_pos[i] = row < nrows ? pos0 + row / p.g : -1;
      row_start[i] = (row < nrows && p.window > 0) ? max(0, row_pos[i] + 1 - p.window) : 0;
    }
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
    for (int t = 0; t < mine_n; ++t) {
      const int s = warp * DEPTH + t % DEPTH;
      // one view of the flag for the whole warp (another warp may set it at any moment)
      const bool gave_up = __shfl_sync(0xffffffffu, (int)*aborted, 0) != 0;
      const bool have = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), (t / DEPTH) & 1,
                                                          gave_up ? DRAIN_LIMIT_NS : WAIT_LIMIT_NS));
      if (!have) {
        // the copies of the tiles already asked for are still waited for, briefly; nothing more is asked for
        if (lane == 0) gb_err::report(ERR_WAIT_FULL);
        *aborted = 1;
        continue;
      }
      uint8_t* ks = ring + s * STAGE_BYTES;
      uint8_t* vs = ks + OPERAND_BYTES;
      const int key0 = (tile_begin + warp + CONSUMERS * t) * TK;
      if (key0 < lo || key0 + TK - 1 > hi) {
        // value rows that no query may read are cleared: 128 bytes per row and half
        for (int e = lane; e < TK * HALVES * 8; e += 32) {
          const int key = (e >> 3) % TK, h = (e >> 3) / TK, c = e & 7;
          if (key0 + key < lo || key0 + key > hi)
            *reinterpret_cast<uint4*>(vs + h * HALF_BYTES + key * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }
      if (!gave_up) {
        process_tile<HD, SwizzledTile<HD, TK>, TK>(st, qf, SwizzledTile<HD, TK>{ks}, SwizzledTile<HD, TK>{vs}, key0, row_pos,
                                                   row_start, p.scale_log2, false);
        __syncwarp();             // every lane is done with the stage before it is filled again
        issue(t + DEPTH);
      }
    }
    // every tile this CTA asked for has arrived and has been used: the ring becomes the merge buffers
    asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
    // ---- the four warps' results into shared memory: [warp][row][RS]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
      st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
      const int row = lane / 4 + 8 * i;
      if (row >= nrows) continue;
      float* dst = red + (warp * ROWS + row) * RS;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + (lane % 4) * 2) = make_float2(st.o[n][2 * i], st.o[n][2 * i + 1]);
      if (lane % 4 == 0) {
        dst[HD] = st.m[i] * p.scale_log2;     // in units of the exponent, as the merges want it
        dst[HD + 1] = st.l[i];
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
    // ---- merge the warps: sixteen threads share a row, each computes the row's weights exp2(m_w - m)
    // itself. A CTA that has the request's keys to itself writes the result; one of several puts its
    // rows into the partial results in global memory.
    float* my_part = CLUSTER ? nullptr : partials + ((size_t)(r * p.Hkv + kvh) * ranks + rank) * (ROWS * RS);
    const bool send = CLUSTER && ranks > 1 && rank != 0;
    const uint32_t remote = send ? map_to_rank(smem_u32(parts) + (uint32_t)(rank - 1) * nrows * RS * 4, 0) : 0;
    const uint32_t remote_bar = send ? map_to_rank(smem_u32(&part_bar), 0) : 0;
    const int sub = threadIdx.x & 15;
    for (int row = threadIdx.x >> 4; row < nrows; row += CTHREADS / 16) {
      float f[CONSUMERS], m = -INFINITY;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, red[(w * ROWS + row) * RS + HD]);
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) {
        const float mw = red[(w * ROWS + row) * RS + HD];
        f[w] = mw == -INFINITY ? 0.f : fast_exp2(mw - m);
      }
      // columns sub, sub + 16, ...; column HD is the maximum, HD + 1 the denominator (weighted like the sums)
      float l = 0.f;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) l += f[w] * red[(w * ROWS + row) * RS + HD + 1];
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g) * HD;
      for (int c = sub; c < RS; c += 16) {
        float v = m;
        if (c != HD) {
          v = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMERS; ++w) v += f[w] * red[(w * ROWS + row) * RS + c];
        }
        if (ranks == 1) {
          if (c < HD) dst[c] = __float2bfloat16_rn(v * inv);
        } else if (!CLUSTER) {
          my_part[row * RS + c] = v;
        } else if (send) {
          st_async_f32(remote + (uint32_t)(row * RS + c) * 4, remote_bar, v);
        } else {
          mine[row * RS + c] = v;
        }
      }
    }
    if (CLUSTER && ranks > 1 && rank == 0) {
      // ---- the cluster's first CTA: its own rows and the others' [rank - 1][nrows][RS], in rank order
      bool got = true;
      if (!mbar_wait(smem_u32(&part_bar), 0)) {
        if (threadIdx.x == 0) gb_err::report(5);
        got = false;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
      for (int row = threadIdx.x >> 4; got && row < nrows; row += CTHREADS / 16) {
        float f[CLUSTER_RANKS], m = mine[row * RS + HD];
        for (int q = 1; q < ranks; ++q) m = fmaxf(m, parts[((q - 1) * nrows + row) * RS + HD]);
        float l = 0.f;
#pragma unroll
        for (int q = 0; q < CLUSTER_RANKS; ++q) {
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
          for (int q = 1; q < CLUSTER_RANKS; ++q)
            if (q < ranks) acc += f[q] * parts[((q - 1) * nrows + row) * RS + c];
          dst[c] = __float2bfloat16_rn(acc * inv);
        }
      }
    }
    if (!CLUSTER && ranks > 1) {
      // ---- the CTA that finishes last merges: every CTA publishes its rows (fence, then a count in
      // global memory); the one that counts the last arrival reads them all back, in rank order, so
      // that the sum is the same whichever CTA it is. It leaves the count at zero for the next launch.
      __shared__ int last_s;
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
      if (threadIdx.x == 0) {
        const int seen = atomicAdd(&counters[r * p.Hkv + kvh], 1);
        last_s = seen == ranks - 1;
        if (last_s) counters[r * p.Hkv + kvh] = 0;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory");
      if (last_s) {
        __threadfence();
        // loads of all ranks' values are asked for together (the loops have a fixed length and are
        // unrolled), so that the merge costs a few trips to L2 and not one per rank
        const float* all = partials + (size_t)(r * p.Hkv + kvh) * ranks * (ROWS * RS);
        for (int row = threadIdx.x >> 4; row < nrows; row += CTHREADS / 16) {
          float f[MAX_RANKS], lq[MAX_RANKS], m = -INFINITY;
#pragma unroll
          for (int q = 0; q < MAX_RANKS; ++q) {
            f[q] = q < ranks ? __ldcg(all + (q * ROWS + row) * RS + HD) : -INFINITY;
            lq[q] = q < ranks ? __ldcg(all + (q * ROWS + row) * RS + HD + 1) : 0.f;
          }
#pragma unroll
          for (int q = 0; q < MAX_RANKS; ++q) m = fmaxf(m, f[q]);
          float l = 0.f;
#pragma unroll
          for (int q = 0; q < MAX_RANKS; ++q) {
            f[q] = f[q] == -INFINITY ? 0.f : fast_exp2(f[q] - m);
            l += f[q] * lq[q];
          }
          const float inv = l > 0.f ? 1.0f / l : 0.f;
          __nv_bfloat16* dst = p.out + ((size_t)(q_begin + row / p.g) * p.Hq + kvh * p.g + row % p.g) * HD;
#pragma unroll
          for (int cc = 0; cc < HD / 16; ++cc) {
            const int c = sub + 16 * cc;
            float v[MAX_RANKS];
#pragma unroll
            for (int q = 0; q < MAX_RANKS; ++q) v[q] = q < ranks ? __ldcg(all + (q * ROWS + row) * RS + c) : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int q = 0; q < MAX_RANKS; ++q) acc += f[q] * v[q];
            dst[c] = __float2bfloat16_rn(acc * inv);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  long long pages;
  int kv_heads, page_size, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && pages == o.pages && kv_heads == o.kv_heads && page_size == o.page_size && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.pages) * 31) ^ (size_t)k.kv_heads * 7919 ^
           (size_t)k.page_size * 104729 ^ (size_t)k.box_rows * 1299709;
  }
};

// A pool [pages][kv heads][page_size][HD] of bfloat16 seen through boxes [1][1][box_rows][64], 128-byte
// swizzle; what lies outside (page -1) reads as zeros.
int pool_map(const void* ptr, long long pages, int kv_heads, int page_size, int box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, pages, kv_heads, page_size, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return GB_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return gb::fail(GB_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)pages};
  cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)HD * 2 * page_size, (cuuint64_t)HD * 2 * page_size * kv_heads};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return gb::fail(GB_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code %d for a cache pool", (int)r);
  if (cache.size() >= 1024) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return GB_OK;
}

}  // namespace

namespace attn {

int decode_tma_max_ranks(bool cluster) { return cluster ? CLUSTER_RANKS : MAX_RANKS; }

bool decode_tma_takes(const Params& p, long long pages) {
  const int ps = p.page_size;
  return pages > 0 && (ps == 8 || ps == 16 || ps == 32 || ps == 64 || ps == 128) && ((uintptr_t)p.k_pool % 16) == 0 &&
         ((uintptr_t)p.v_pool % 16) == 0 && ((uintptr_t)p.q % 4) == 0 && encode_fn() != nullptr;
}

// scratch: COUNTER_BYTES of counters (zero before the first launch; every launch leaves them zero),
// then the partial results [R][kv heads][ranks][16][head_dim + 2] floats. With less scratch than
// `ranks` CTAs per request need, fewer share a request's keys (one needs none).
long long decode_tma_scratch_bytes(int R, int kv_heads, int ranks) {
  return ranks <= 1 ? 0 : COUNTER_BYTES + (long long)R * kv_heads * ranks * ROWS * RS * 4;
}

int launch_decode_tma(const Params& p, long long pages, int R, int ranks, bool cluster, void* scratch,
                      long long scratch_bytes, cudaStream_t stream) {
  ranks = ranks < 1 ? 1 : (ranks > MAX_RANKS ? MAX_RANKS : ranks);
  if (cluster) {
    if (ranks > CLUSTER_RANKS) ranks = CLUSTER_RANKS;
  } else {
    if ((long long)R * p.Hkv * 4 > COUNTER_BYTES || ((uintptr_t)scratch & 15) != 0) ranks = 1;
    while (ranks > 1 && (scratch == nullptr || decode_tma_scratch_bytes(R, p.Hkv, ranks) > scratch_bytes)) --ranks;
  }
  const int box_rows = p.page_size < TK ? p.page_size : TK;
  CUtensorMap km, vm;
  int rc = pool_map(p.k_pool, pages, p.Hkv, p.page_size, box_rows, &km);
  if (rc) return rc;
  rc = pool_map(p.v_pool, pages, p.Hkv, p.page_size, box_rows, &vm);
  if (rc) return rc;
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e1 = cudaFuncSetAttribute(attention_decode_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaError_t e2 = cudaFuncSetAttribute(attention_decode_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          smem_cluster(CLUSTER_RANKS));
    if (e1 != cudaSuccess || e2 != cudaSuccess)
      return gb::fail(GB_CUDA_ERROR, "attention (decode, TMA): %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    configured.done();
  }
  if (cluster && ranks > 1) {
    float* none = nullptr;
    int* no_counters = nullptr;
    return gb::check_pdl_launch(gb::launch_pdl(attention_decode_tma_kernel<true>, dim3(ranks, p.Hkv, R), dim3(THREADS),
                                               smem_cluster(ranks), stream, dim3(ranks, 1, 1), km, vm, p, box_rows, none,
                                               no_counters),
                                "attention (decode, TMA, clusters)");
  }
  int* counters = reinterpret_cast<int*>(scratch);
  float* partials = ranks > 1 ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + COUNTER_BYTES) : nullptr;
  return gb::check_pdl_launch(gb::launch_pdl(attention_decode_tma_kernel<false>, dim3(ranks, p.Hkv, R), dim3(THREADS), SMEM_BYTES,
                                             stream, dim3(1, 1, 1), km, vm, p, box_rows, partials, counters),
                              "attention (decode, TMA)");
}

int decode_tma_error_check() { return gb_err::fetch_and_clear(); }
int decode_tma_set_error_sink(int* host_word) { return gb_err::set_sink(host_word); }

}  // namespace attn

#else  // other head sizes: the kernel with per-thread copies

namespace attn {
int decode_tma_max_ranks(bool) { return 0; }
bool decode_tma_takes(const Params&, long long) { return false; }
long long decode_tma_scratch_bytes(int, int, int) { return 0; }
int launch_decode_tma(const Params&, long long, int, int, bool, void*, long long, cudaStream_t) {
  return gb::fail(GB_UNSUPPORTED, "attention (decode, TMA): head size %d", GB_HEAD_DIM);
}
int decode_tma_error_check() { return 0; }
int decode_tma_set_error_sink(int*) { return 0; }
}  // namespace attn

#endif
