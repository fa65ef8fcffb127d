// Causal grouped-query attention over the paged cache for prompt portions on the
// fifth-generation tensor cores: both matrix products of a tile are tcgen05.mma with
// accumulators in tensor memory, operands arrive by TMA, the softmax runs in 32-bit in
// registers between them, and the probabilities go back into tensor memory, where the second
// product reads them.
//
// garuda/src/llama/mod.rs:793-818: s_j = dot(q, K_j) * scale over keys [start, pos],
// softmax with the maximum subtracted, sum of p_j V_j; query head h reads kv head h / g;
// start = max(0, pos + 1 - window) with a window (garuda/src/cache/mod.rs:333-338).
//
// A piece of work is 128 query rows, (token, head-of-group) pairs that share one kv head of one
// request; its keys are walked in tiles of 128. The kernel is persistent: one CTA per SM takes
// pieces until none are left (rounds of gridDim.x pieces, walked forth and back so that long and
// short ones mix), keeping its tensor memory and barriers; the queries and first keys of the next
// piece arrive, and its first S products run, while the last tiles of the one before are in the
// softmax.
//   warp 0   TMA. The query tile (3-D boxes [tokens][group][64], two buffers); per key tile one
//            4-D box per page and block of 64 channels, keys and values in rings of their own
//            (keys are needed two tiles before their values). The lanes look up the pages of
//            several tiles in one round trip and issue one page's copies each.
//   warp 1   one lane: O += P V of the tile whose softmax just ended (P from tensor memory, V as
//            it lies in the cache, keys along the rows: an MN-major operand), one accumulator per
//            group for the whole piece; then S = Q K^T for the tile two ahead into the S buffer
//            that this tile's P has just been read from. This warp is the one the tensor cores
//            wait for, so it steps counters instead of dividing, advances descriptors made once,
//            and learns the pieces' lengths 32 at a time from its lanes.
//   warps 2-9  two groups of 128 threads; a thread owns a query row and its group's 64 keys of
//            every tile, an attention stream of its own: reads its 64 scores from tensor memory,
//            masks (only on tiles that touch a row's limits), exp2 with the scale folded in
//            against a reference maximum, writes P in bfloat16 over the first half of the scores
//            it has read. The reference maximum follows the running maximum only when that has
//            grown by more than 2^8 for some row of the warp; only then is the accumulator in
//            tensor memory rescaled (read, multiplied, written back). The result is the same
//            quotient, and probabilities stay below 2^8. At the end of a piece the two groups'
//            streams are merged, each group writing half of the channels. The groups also clear
//            the value rows no query may read (a stray NaN times a zero probability would
//            spoil a sum), and one of their threads tells the TMA warp which stages the tensor
//            core has finished with (a commit costs the issuing thread as much as two products).
// Tensor memory (512 columns): two S buffers of 128 columns (group g's scores, then its
// probabilities, at g * 64), and one accumulator of `head size` columns per group.
// Measured on this hardware: a product with fewer than 128 columns costs as much as one with 128
// (about 70 cycles for M = 128, K = 16), which is why S is one 128-column product for both groups.
// Every wait is bounded; a wait that runs out sets the error word and the CTA winds down.
//
// Built for head sizes 64 and 128 (one or two 128-byte swizzled rows per key); other head sizes use
// the mma.sync kernels.
#include "attention_common.cuh"
#include "error_word.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 64
#endif

#if GB_HEAD_DIM == 64 || GB_HEAD_DIM == 128

namespace {

using namespace tc;
using attn::Params;

constexpr int HD = GB_HEAD_DIM;
constexpr int BLOCKS = HD / 64;     // blocks of 64 channels: one swizzled 128-byte row each
constexpr int QROWS = 128;          // query rows per CTA
constexpr int KT = 128;             // keys per tile
constexpr int GROUPS = 2;           // softmax groups: each walks its own half of every key tile
constexpr int GK = KT / GROUPS;     // keys per group and tile
constexpr int ROW_BYTES = 128;      // one swizzled row: 64 channels
constexpr int BLOCK_BYTES = 128 * ROW_BYTES;        // 128 rows (queries or keys) of one block of channels
constexpr int Q_BYTES = BLOCKS * BLOCK_BYTES, K_BYTES = Q_BYTES, V_BYTES = Q_BYTES;
constexpr int K_STAGES = HD == 64 ? 4 : 2;          // keys live from their S product's issue to its end
constexpr int V_STAGES = HD == 64 ? 5 : 3;          // values until P V, two tiles later
constexpr int TILE_BYTES = 2 * Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int S_BUFS = 2;                           // S buffers: the S products run this many tiles ahead
constexpr int O_COL0 = S_BUFS * KT;                 // behind the S buffers
// Who tells the TMA warp that a stage of keys is free: with few stages the tensor core itself, as
// soon as the S product has ended (a commit costs the issuing thread as much as two products);
// with more, a softmax thread once it has seen the S buffer.
constexpr bool KEYS_FREED_BY_COMMIT = K_STAGES < S_BUFS + 1;
constexpr int THREADS = 64 + GROUPS * 128;
constexpr float RESCALE_ABOVE = 8.f;                // in powers of two
static_assert(GK == 64 && O_COL0 + GROUPS * HD <= TMEM_COLS, "tensor memory layout");
constexpr int CH = HD / GROUPS;     // channels that a group writes out in the merge
constexpr int ML_BUFS = HD == 64 ? 2 : 1;   // copies of the groups' maxima and denominators (shared memory is short with head size 128)

// Barriers and the like, behind the tiles in dynamic shared memory.
struct Misc {
  uint64_t q_full[2], q_empty[2], k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
  uint64_t s_ready[S_BUFS], p_ready[S_BUFS], o_ready;
  uint32_t tmem_base;
  int abort;
  float2 ml[ML_BUFS][GROUPS][QROWS];     // the groups' reference maxima and denominators, for the merge
};
constexpr int SMEM_BYTES = TILE_BYTES + (int)sizeof(Misc);
static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The largest of three in one instruction.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// One piece of work: 128 query rows of one request and kv head.
struct Item {
  bool valid;
  int kvh, q_begin, tok0, nrows, pos0, lo, hi, tile_begin, n_tiles;
  const int32_t* table;
};

// Items are numbered request by request, the tiles of a request from its end (the longest first), the
// kv heads innermost. A CTA takes every gridDim.x-th item, so each gets long and short ones.
__device__ __forceinline__ Item decode_item(const Params& p, int q_tiles, int item) {
  Item w;
  const int per_req = q_tiles * p.Hkv;
  const int r = item / per_req, rem = item % per_req;
  const int qt = q_tiles - 1 - rem / p.Hkv;
  w.kvh = rem % p.Hkv;
  // The batch's lengths and block tables were copied in before the step's first kernel.
  w.q_begin = p.cu_q[r];
  const int q_len = p.cu_q[r + 1] - w.q_begin;
  const int tokens_per_tile = QROWS / p.g;
  w.tok0 = qt * tokens_per_tile;
  w.valid = q_len * p.g > attn::ROWS_DECODE && w.tok0 < q_len;      // else a decode request, or past its end
  const int kv_len = p.kv_lens[r];
  const int ntok = min(tokens_per_tile, q_len - w.tok0);
  w.nrows = ntok * p.g;
  w.pos0 = kv_len - q_len + w.tok0;                                 // position of the tile's first token
  w.lo = p.window > 0 ? max(0, w.pos0 + 1 - p.window) : 0;          // first key any row reads
  w.hi = w.pos0 + ntok - 1;                                         // last key any row reads
  w.tile_begin = w.lo / KT;
  w.n_tiles = w.valid ? w.hi / KT + 1 - w.tile_begin : 0;
  w.table = p.block_table + (size_t)r * p.table_width;
  return w;
}

// Walks this CTA's items tile by tile.
// The k-th item of this CTA: rounds of gridDim.x items, walked forth and back in turn, so that the
// CTA that got the longest item of one round gets the shortest of the next.
__device__ __forceinline__ int cta_item(int k) {
  const int g = (int)gridDim.x, b = (int)blockIdx.x;
  return k * g + ((k & 1) ? g - 1 - b : b);
}

struct Cursor {
  int item, total, step, q_tiles, round;
  int it;          // valid items before this one
  int j;           // tile within the item
  Item w;
  bool done;
  __device__ __forceinline__ void seek(const Params& p) {
    done = true;
    while ((long long)round * step < total) {       // a round may end before this CTA's place in it
      if (item < total) {
        w = decode_item(p, q_tiles, item);
        if (w.valid) { done = false; break; }
      }
      item = cta_item(++round);
    }
  }
  __device__ __forceinline__ void start(const Params& p, int q_tiles_, int total_) {
    round = 0, step = gridDim.x, total = total_, q_tiles = q_tiles_, it = 0, j = 0;
    item = cta_item(0);
    seek(p);
  }
  __device__ __forceinline__ void next_item(const Params& p) {
    item = cta_item(++round), ++it, j = 0;
    seek(p);
  }
};

// The same walk for the warp that issues the matrix products: it needs nothing of an item but its
// number of tiles, and everything it executes delays the tensor cores. Its lanes decode 32 items at
// a time, one each; the walk then only shuffles the counts out.
struct TileWalk {
  int base;        // this CTA's items before the batch
  int my_n;        // tiles of this lane's item of the batch (0: none, or not a valid item)
  int lane_i;      // the current item's lane
  int n, j;        // the current item's tiles, the current tile
  int it;          // valid items before the current one
  bool done;
  __device__ __forceinline__ void load(const Params& p, int q_tiles, int total) {
    const int k = base + (int)(threadIdx.x & 31);
    const long long item = (long long)k * gridDim.x < total ? cta_item(k) : total;
    my_n = item < total ? decode_item(p, q_tiles, (int)item).n_tiles : 0;
  }
  __device__ __forceinline__ void seek(const Params& p, int q_tiles, int total) {
    for (;;) {
      // the next lane of the batch with tiles, if any
      const unsigned have = __ballot_sync(0xffffffffu, my_n > 0) & (0xffffffffu << lane_i);
      if (lane_i < 32 && have != 0) {
        lane_i = __ffs(have) - 1;
        n = __shfl_sync(0xffffffffu, my_n, lane_i);
        return;
      }
      base += 32;
      lane_i = 0;
      if ((long long)base * gridDim.x >= total) {
        done = true;
        return;
      }
      load(p, q_tiles, total);
    }
  }
  __device__ __forceinline__ void start(const Params& p, int q_tiles, int total) {
    base = 0, lane_i = 0, j = 0, it = 0, n = 0, done = false;
    load(p, q_tiles, total);
    seek(p, q_tiles, total);
  }
  __device__ __forceinline__ void next_tile(const Params& p, int q_tiles, int total) {
    if (++j >= n) {
      j = 0, ++it, ++lane_i;
      if (lane_i >= 32) lane_i = 32;
      seek(p, q_tiles, total);
    }
  }
};

// A persistent kernel: one CTA per SM takes items until none are left, keeping its tensor memory and
// barriers, so that the queries and first keys of the next item arrive, and its first S products
// run, while the last tiles of the one before are still in the softmax.
__global__ void __launch_bounds__(THREADS, 1)
attention_tile_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map, const Params p, const int q_tiles,
                         const int total_items) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Misc& mc = *reinterpret_cast<Misc*>(smem_raw + TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_s = smem_u32(smem_raw);                         // two query buffers
  const uint32_t k_s = q_s + 2 * Q_BYTES;                          // key stage s at k_s + s * K_BYTES
  const uint32_t v_s = k_s + K_STAGES * K_BYTES;                   // value stage s at v_s + s * V_BYTES
  if ((q_s & 1023u) != 0) {                                        // the swizzle needs it; never seen
    if (threadIdx.x == 0) gb_err::report(ERR_WAIT_DRAIN);
    return;
  }

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&mc.q_full[b]), 1);
      mbar_init(smem_u32(&mc.q_empty[b]), 1);
    }
    for (int b = 0; b < S_BUFS; ++b) {
      mbar_init(smem_u32(&mc.s_ready[b]), 1);
      mbar_init(smem_u32(&mc.p_ready[b]), GROUPS * 128);
    }
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(smem_u32(&mc.k_full[s]), 1);
      mbar_init(smem_u32(&mc.k_empty[s]), 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(smem_u32(&mc.v_full[s]), 1);
      mbar_init(smem_u32(&mc.v_empty[s]), 1);
    }
    mbar_init(smem_u32(&mc.o_ready), 1);
    mc.abort = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&q_map);
    prefetch_tensormap(&k_map);
    prefetch_tensormap(&v_map);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&mc.tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = mc.tmem_base;
  volatile int* abort_s = &mc.abort;
  gb::pdl_launch_dependents();
  gb::pdl_wait();      // queries and this step's keys and values come from the kernel in front

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA
    // The whole warp: its lanes look up the pages of the next 32 / pages_per_tile tiles in one
    // round trip (a lookup per tile by one thread, each waited for, was what the kernel's pace
    // hung on); for a tile, lane g issues the copies of the tile's g-th page; lane 0 waits for
    // the stages and tells their barriers how many bytes to expect.
    const int page_shift = __ffs(p.page_size) - 1;         // pages are a power of two of keys
    const int pages_per_tile = KT >> page_shift;           // 1 to 16
    const int tiles_per_batch = 32 / pages_per_tile;
    const uint32_t page_bytes = (uint32_t)p.page_size * ROW_BYTES;     // of one block of channels
    int gt = 0;                       // tiles so far, over all items
    int ks = 0, kpar = 1;             // the key stage to fill and the phase of its "empty" barrier to wait for
    int vs = 0, vpar = 1;             // the same for values
    bool ok = true;
    Cursor c;
    for (c.start(p, q_tiles, total_items); !c.done && ok; c.next_item(p)) {
      const Item& w = c.w;
      const int qb = c.it & 1;
      if (lane == 0) {
        if (c.it >= 2 && !mbar_wait(smem_u32(&mc.q_empty[qb]), ((c.it >> 1) & 1) ^ 1)) {
          gb_err::report(ERR_WAIT_EMPTY);
          *abort_s = 1;
        }
        if (!*abort_s) {
          mbar_arrive_expect_tx(smem_u32(&mc.q_full[qb]), Q_BYTES);
#pragma unroll
          for (int h = 0; h < BLOCKS; ++h)
            tma_load_3d(q_s + qb * Q_BYTES + h * BLOCK_BYTES, &q_map, smem_u32(&mc.q_full[qb]), h * 64, w.kvh * p.g,
                        w.q_begin + w.tok0);
        }
      }
      int entry = -1;       // this lane's page of the batch: tile lane / pages_per_tile, page lane % pages_per_tile
      for (int j = 0; j < w.n_tiles && ok; ++j, ++gt) {
        const int jb = j % tiles_per_batch;
        if (jb == 0) {
          // pages that hold a key some row reads, and exist
          const int first = (w.tile_begin + j) * KT + lane * p.page_size;
          entry = (first <= w.hi && first + p.page_size > w.lo) ? w.table[first >> page_shift] : -1;
        }
        const int page = __shfl_sync(0xffffffffu, entry, (jb * pages_per_tile + lane) & 31);
        const bool mine = lane < pages_per_tile && page >= 0;
        const int count = __popc(__ballot_sync(0xffffffffu, mine));
        // keys first: their product runs two tiles before the values' one
        if (lane == 0) {
          if (gt >= K_STAGES && !mbar_wait(smem_u32(&mc.k_empty[ks]), kpar)) {
            gb_err::report(ERR_WAIT_EMPTY);
            *abort_s = 1;
          }
          if (!*abort_s) {
            if (count == 0) mbar_arrive(smem_u32(&mc.k_full[ks]));
            else mbar_arrive_expect_tx(smem_u32(&mc.k_full[ks]), (uint32_t)BLOCKS * count * page_bytes);
          }
        }
        __syncwarp();
        if (*abort_s) { ok = false; break; }
        if (mine) {
#pragma unroll
          for (int h = 0; h < BLOCKS; ++h)
            tma_load_4d(k_s + ks * K_BYTES + h * BLOCK_BYTES + lane * page_bytes, &k_map, smem_u32(&mc.k_full[ks]), h * 64, 0,
                        w.kvh, page);
        }
        if (lane == 0) {
          if (gt >= V_STAGES && !mbar_wait(smem_u32(&mc.v_empty[vs]), vpar)) {
            gb_err::report(ERR_WAIT_EMPTY);
            *abort_s = 1;
          }
          if (!*abort_s) {
            if (count == 0) mbar_arrive(smem_u32(&mc.v_full[vs]));
            else mbar_arrive_expect_tx(smem_u32(&mc.v_full[vs]), (uint32_t)BLOCKS * count * page_bytes);
          }
        }
        __syncwarp();
        if (*abort_s) {
          ++gt;       // this tile's keys are in flight
          ok = false;
          break;
        }
        if (mine) {
#pragma unroll
          for (int h = 0; h < BLOCKS; ++h)
            tma_load_4d(v_s + vs * V_BYTES + h * BLOCK_BYTES + lane * page_bytes, &v_map, smem_u32(&mc.v_full[vs]), h * 64, 0,
                        w.kvh, page);
        }
        if (++ks == K_STAGES) ks = 0, kpar ^= 1;
        if (++vs == V_STAGES) vs = 0, vpar ^= 1;
      }
      __syncwarp();
      if (*abort_s) ok = false;
    }
    if (*abort_s && lane == 0) {
      // wind down: let the copies in flight land before the CTA's shared memory is given up.
      // (A tile counted in gt whose values were not asked for has a barrier that nothing
      // completes; its wait runs out after 20 ms.)
      auto drain = [&](uint64_t* bars, int stages) {
        for (int t = gt > stages ? gt - stages : 0; t < gt; ++t) {
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&bars[t % stages]), (t / stages) & 1)) {
            if (globaltimer_ns() - t0 > 20000000ull) {  // 20 ms
              gb_err::report(ERR_WAIT_DRAIN);
              break;
            }
          }
        }
      };
      drain(mc.k_full, K_STAGES);
      drain(mc.v_full, V_STAGES);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    // The S products run two tiles ahead of the P V products, across the items' borders. Whatever
    // this warp executes between two products delays the tensor cores, so it is kept short: stage
    // and buffer counters are stepped, not divided; descriptors are made once and advanced. On
    // this hardware a product with fewer than 128 columns takes as long as one with 128 (about
    // 70 cycles for M = 128, K = 16), so S is computed for both groups at once (their S buffers
    // lie side by side). After a tile's softmax its P V goes first: it reads the probabilities
    // from the S buffer that the S product two tiles ahead then overwrites (products run in the
    // order of their issue).
    constexpr uint32_t idesc_s = instr_desc_bf16(QROWS, KT);
    constexpr uint32_t idesc_o = instr_desc_bf16(QROWS, HD) | INSTR_B_MN_MAJOR;
    const uint64_t dq0 = smem_desc_sw128(q_s), dk0 = smem_desc_sw128(k_s),
                   dv0 = smem_desc_sw128_mn(v_s, BLOCKS > 1 ? BLOCK_BYTES : 16);
    bool ok = true;
    TileWalk ws, wp;               // the S products' tile, the P V products' tile
    ws.start(p, q_tiles, total_items);
    wp = ws;
    int k_stage = 0, k_par = 0;                    // key stage (and its phase) of the S tile
    int v_stage = 0, v_par = 0;                    // value stage of the P V tile
    int s_buf = 0;                                 // S buffer of the S tile
    int p_buf = 0, p_par = 0;                      // buffer of the P V tile and its phase
    auto issue_s = [&]() {      // S = Q K^T of the S tile into S buffer s_buf (both groups' columns)
      const int qb = ws.it & 1;
      if (ws.j == 0 && !mbar_wait(smem_u32(&mc.q_full[qb]), (ws.it >> 1) & 1)) ok = false;
      if (ok && !mbar_wait(smem_u32(&mc.k_full[k_stage]), k_par)) ok = false;
      if (!ok) {
        if (lane == 0) gb_err::report(ERR_WAIT_FULL);
        return;
      }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int h = 0; h < BLOCKS; ++h)
          mma_bf16_x4(tmem_base + s_buf * KT, dq0 + (uint64_t)(qb * (Q_BYTES >> 4) + h * (BLOCK_BYTES >> 4)),
                      dk0 + (uint64_t)(k_stage * (K_BYTES >> 4) + h * (BLOCK_BYTES >> 4)), idesc_s, 2, 2, h > 0);
        mma_commit(smem_u32(&mc.s_ready[s_buf]));      // the softmax warps pass it on to the queries' "empty" barrier
        if (KEYS_FREED_BY_COMMIT) mma_commit(smem_u32(&mc.k_empty[k_stage]));
      }
      __syncwarp();
      if (++k_stage == K_STAGES) k_stage = 0, k_par ^= 1;
      if (++s_buf == S_BUFS) s_buf = 0;
      ws.next_tile(p, q_tiles, total_items);
    };
#pragma unroll 1
    for (int b = 0; b < S_BUFS; ++b)
      if (ok && !ws.done) issue_s();
    while (ok && !wp.done) {
      if (*abort_s) break;
      if (ok && !mbar_wait(smem_u32(&mc.p_ready[p_buf]), p_par)) {
        if (lane == 0) gb_err::report(ERR_WAIT_ACCUM);
        ok = false;
      }
      if (ok && !mbar_wait(smem_u32(&mc.v_full[v_stage]), v_par)) {
        if (lane == 0) gb_err::report(ERR_WAIT_FULL);
        ok = false;
      }
      if (!ok) break;
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < GROUPS; ++g)
          mma_bf16_ts<GK / 16>(tmem_base + O_COL0 + g * HD, tmem_base + p_buf * KT + g * GK,
                         dv0 + (uint64_t)(v_stage * (V_BYTES >> 4) + g * (GK * ROW_BYTES >> 4)), idesc_o,
                         16 * ROW_BYTES >> 4, wp.j > 0);
        mma_commit(smem_u32(&mc.o_ready));             // the softmax warps pass it on to the values' "empty" barrier
      }
      __syncwarp();
      // both groups have read this S buffer in full, and the products above read their P from it
      // before the next one writes: the S product two tiles ahead takes the buffer over
      if (!ws.done) issue_s();
      if (!ok) break;
      if (++v_stage == V_STAGES) v_stage = 0, v_par ^= 1;
      if (++p_buf == S_BUFS) p_buf = 0, p_par ^= 1;
      wp.next_tile(p, q_tiles, total_items);
    }
    if (!ok) *abort_s = 1;
  } else {
    // -------------------------------------------------------------------- softmax warps
    // Group g takes keys [g * 64, g * 64 + 64) of every tile: an attention stream of its own
    // (reference maximum, denominator, accumulator), merged with the other group's at the end.
    // Two groups put two warps on every scheduler, so that one computes while the other waits
    // for tensor memory.
    const int grp = (warp - 2) >> 2;
    const int quarter = warp & 3;                        // the TMEM lanes this warp may read
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t o_mine = lane_addr + O_COL0 + grp * HD;
    const float scale_log2 = p.scale_log2;
    bool ok = true;       // false: this thread only keeps the others company at the barriers
    int gt = 0;           // tiles so far, over all items
    int sb = 0, sph = 0;          // the current tile's S buffer and the phase of its barriers
    int kstage = 0;               // the current tile's stage of keys
    int vstage = 0, vpar = 0;     // the current tile's stage of values and its phase
    int vprev = 0;                // the stage of the tile before
    const bool passes_on = threadIdx.x == 64;      // one thread tells the TMA warp what the tensor core has finished with
    Cursor c;
    for (c.start(p, q_tiles, total_items); !c.done; c.next_item(p)) {
      const Item& w = c.w;
      const int row_pos = row < w.nrows ? w.pos0 + row / p.g : -1;       // no key is valid for a padding row
      const int row_start = (row < w.nrows && p.window > 0) ? max(0, row_pos + 1 - p.window) : 0;
      float m = -INFINITY, l = 0.f;      // m: the reference maximum of the raw dot products

      // waits until the P V products of the tile counted t have ended
      auto wait_o = [&](int t) {
        if (!mbar_wait(smem_u32(&mc.o_ready), t & 1)) {
          if (lane == 0) gb_err::report(ERR_WAIT_ACCUM);
          ok = false;
          *abort_s = 1;
        }
        tc_fence_after_sync();
      };

      for (int j = 0; j < w.n_tiles && ok; ++j, ++gt) {
        if (*abort_s) { ok = false; break; }
        if (!mbar_wait(smem_u32(&mc.s_ready[sb]), sph)) {
          if (lane == 0) gb_err::report(ERR_WAIT_ACCUM);
          ok = false;
          *abort_s = 1;
          break;
        }
        tc_fence_after_sync();
        if (passes_on) {      // S of this tile is complete: its keys have been read, and after an item's last tile its queries
          if (!KEYS_FREED_BY_COMMIT) mbar_arrive(smem_u32(&mc.k_empty[kstage]));
          if (j == w.n_tiles - 1) mbar_arrive(smem_u32(&mc.q_empty[c.it & 1]));
        }
        if (++kstage == K_STAGES) kstage = 0;
        const uint32_t s_addr = lane_addr + sb * KT + grp * GK;
        // the row's 64 scores of this group, one wait for the two loads
        uint32_t sv[GK / 32][32];
#pragma unroll
        for (int h = 0; h < GK / 32; ++h) tmem_ld_32(s_addr + h * 32, sv[h]);
        const int tile_key0 = (w.tile_begin + j) * KT;
        const bool edge = tile_key0 < w.lo || tile_key0 + KT - 1 > w.hi;
        if (edge) {
          // Value rows that no row may read hold whatever was there (a page that was not fetched,
          // the unwritten end of the last page): their probabilities are zero, but zero times a
          // stray NaN is not. Clear them, once the stage's copies have landed: half of each
          // group's threads take one of the group's 64 rows each. (The tensor core reads the
          // values only after this thread's arrival below.)
          if (!mbar_wait(smem_u32(&mc.v_full[vstage]), vpar)) {
            if (lane == 0) gb_err::report(ERR_WAIT_FULL);
            ok = false;
            *abort_s = 1;
          }
          if (ok && row < GK) {
            const int vrow = grp * GK + row, key = tile_key0 + vrow;
            if (key < w.lo || key > w.hi) {
#pragma unroll
              for (int h = 0; h < BLOCKS; ++h) {
                const uint32_t vaddr = v_s + vstage * V_BYTES + h * BLOCK_BYTES + vrow * ROW_BYTES;
#pragma unroll
                for (int ch = 0; ch < ROW_BYTES / 16; ++ch) st_shared_v4(vaddr + ch * 16, 0u, 0u, 0u, 0u);
              }
            }
          }
          fence_proxy_async();            // the tensor core reads the values through the async proxy
        }
        const int vcur = vstage;
        if (++vstage == V_STAGES) vstage = 0, vpar ^= 1;
        tmem_ld_wait();
        if (!ok) break;
        auto sc = [&](int ch) -> float& { return reinterpret_cast<float&>(sv[ch >> 5][ch & 31]); };
        const int key0 = tile_key0 + grp * GK;
        // the keys need no mask if they lie wholly before the first row's position and inside the
        // last row's window
        const bool full = key0 + GK - 1 <= w.pos0 && (p.window <= 0 || key0 >= w.hi + 1 - p.window);
        if (!full) {
#pragma unroll
          for (int ch = 0; ch < GK; ++ch)
            if (!(key0 + ch >= row_start && key0 + ch <= row_pos)) sc(ch) = -INFINITY;
        }
        // four independent chains for the maximum and for the sum
        float mx[4] = {m, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int ch = 0; ch < GK; ch += 8) {
#pragma unroll
          for (int e = 0; e < 4; ++e) mx[e] = max3(mx[e], sc(ch + e), sc(ch + 4 + e));
        }
        const float m_new = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        // The reference maximum moves only if some row of the warp has outgrown it by more than
        // 2^8; then the warp rescales what it has accumulated (the loads and stores of tensor
        // memory are the whole warp's). A row that has seen no valid key yet has nothing to rescale.
        const bool grown = m != -INFINITY && (m_new - m) * scale_log2 > RESCALE_ABOVE;
        bool waited = false;
        if (j > 0 && __any_sync(0xffffffffu, grown)) {
          wait_o(gt - 1);
          waited = true;
          if (!ok) break;
          const float corr = m == -INFINITY ? 1.f : fast_exp2((m - m_new) * scale_log2);
#pragma unroll
          for (int h = 0; h < HD / 32; ++h) {
            uint32_t v[32];
            tmem_ld_32(o_mine + h * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int ch = 0; ch < 32; ++ch) v[ch] = __float_as_uint(__uint_as_float(v[ch]) * corr);
            tmem_st_32(o_mine + h * 32, v);
          }
          l *= corr;
          m = m_new;
        } else if (m == -INFINITY) {
          m = m_new;
        }
        const float neg_m = m == -INFINITY ? 0.f : -m * scale_log2;       // nothing valid yet: avoid inf - inf
        // All exponentials first, in place (the unit that computes them takes a warp's instruction
        // every eight cycles; the multiply-adds in front fit in between), then sums and packing.
#pragma unroll
        for (int ch = 0; ch < GK; ++ch) {
          sc(ch) = fast_exp2(fmaf(sc(ch), scale_log2, neg_m));   // exp2(-inf) = 0 for masked keys
        }
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[GK / 2];
#pragma unroll
        for (int ch = 0; ch < GK; ch += 2) {
          ls[(ch >> 1) & 3] += sc(ch) + sc(ch + 1);
          pk[ch >> 1] = pack_bf16(sc(ch), sc(ch + 1));
        }
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        tmem_st(s_addr, pk);            // over the first half of the scores just read
        tmem_st_wait();
        if (j > 0 && !waited) wait_o(gt - 1);      // every phase of the barrier is seen, in order
        tc_fence_before_sync();         // this thread's accesses to tensor memory are over
        mbar_arrive(smem_u32(&mc.p_ready[sb]));
        if (passes_on && j > 0) mbar_arrive(smem_u32(&mc.v_empty[vprev]));      // the tile before: its P V has ended
        vprev = vcur;
        if (++sb == S_BUFS) sb = 0, sph ^= 1;
      }
      if (ok && w.n_tiles > 0) {
        wait_o(gt - 1);
        if (passes_on && ok) mbar_arrive(smem_u32(&mc.v_empty[vprev]));
      }
      // ---- merge the groups: each writes its share of the channels, summed over all accumulators
      const int mb = ML_BUFS == 2 ? (c.it & 1) : 0;
      mc.ml[mb][grp][row] = make_float2(m, l);
      tc_fence_before_sync();
      asm volatile("bar.sync 1, %0;" ::"n"(GROUPS * 128) : "memory");
      tc_fence_after_sync();
      if (ok && !*abort_s) {
        float a[GROUPS];
        float mt = -INFINITY, lt = 0.f;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) mt = fmaxf(mt, mc.ml[mb][g][row].x);
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
          const float2 x = mc.ml[mb][g][row];
          a[g] = x.x == -INFINITY ? 0.f : fast_exp2((x.x - mt) * scale_log2);
          lt += x.y * a[g];
        }
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
        __nv_bfloat16* dst = p.out + ((size_t)(w.q_begin + w.tok0 + row / p.g) * p.Hq + w.kvh * p.g + row % p.g) * HD + grp * CH;
#pragma unroll
        for (int h = 0; h < CH / 16; ++h) {
          float t[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) t[e] = 0.f;
#pragma unroll
          for (int g = 0; g < GROUPS; g += 2) {      // two accumulators at a time (registers)
            uint32_t v[2][16];
            tmem_ld_16(lane_addr + O_COL0 + g * HD + grp * CH + h * 16, v[0]);
            tmem_ld_16(lane_addr + O_COL0 + (g + 1) * HD + grp * CH + h * 16, v[1]);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) {      // a stream without a valid key has an accumulator that means nothing
              t[e] += a[g] > 0.f ? __uint_as_float(v[0][e]) * (a[g] * inv) : 0.f;
              t[e] += a[g + 1] > 0.f ? __uint_as_float(v[1][e]) * (a[g + 1] * inv) : 0.f;
            }
          }
          if (row < w.nrows) {
            uint4 w0, w1;
            w0.x = pack_bf16(t[0], t[1]), w0.y = pack_bf16(t[2], t[3]), w0.z = pack_bf16(t[4], t[5]), w0.w = pack_bf16(t[6], t[7]);
            w1.x = pack_bf16(t[8], t[9]), w1.y = pack_bf16(t[10], t[11]), w1.z = pack_bf16(t[12], t[13]), w1.w = pack_bf16(t[14], t[15]);
            *reinterpret_cast<uint4*>(dst + h * 16) = w0;
            *reinterpret_cast<uint4*>(dst + h * 16 + 8) = w1;
          }
        }
      }
      // The next item's first P V overwrites the accumulators; it is issued only after all groups
      // have arrived for that tile, that is after all are through here. With one copy of `ml` a
      // group must not write the next item's values while another still reads these.
      if (ML_BUFS == 1) asm volatile("bar.sync 1, %0;" ::"n"(GROUPS * 128) : "memory");
      tc_fence_before_sync();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side
using tc_host::encode_fn;
using tc_host::EncodeTiledFn;

struct MapKey {
  const void* ptr;
  long long d1, d2, d3;
  int b1, b2;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d1 == o.d1 && d2 == o.d2 && d3 == o.d3 && b1 == o.b1 && b2 == o.b2;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.d1) * 31) ^ (std::hash<long long>()(k.d2) * 131) ^
           (std::hash<long long>()(k.d3) * 521) ^ (size_t)k.b1 * 7919 ^ (size_t)k.b2 * 104729;
  }
};

// A bf16 tensor [d3][d2][d1][head size] (channels contiguous) seen through boxes [1][b2][b1][64]
// (d3 = 0: three dimensions, box [b2][b1][64]), 128-byte swizzle; elements outside read as zeros.
int tensor_map(const void* ptr, long long d1, long long d2, long long d3, int b1, int b2, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, d1, d2, d3, b1, b2};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return GB_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return gb::fail(GB_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  const int rank = d3 > 0 ? 4 : 3;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)d1, (cuuint64_t)d2, (cuuint64_t)(d3 > 0 ? d3 : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)HD * 2 * d1, (cuuint64_t)HD * 2 * d1 * d2};
  cuuint32_t box[4] = {64, (cuuint32_t)b1, (cuuint32_t)b2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return gb::fail(GB_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code %d for an attention operand", (int)r);
  if (cache.size() >= 512) cache.clear();      // the query map changes with the number of tokens
  cache.emplace(key, m);
  *out = m;
  return GB_OK;
}

}  // namespace

namespace attn {

bool tile_tc_takes(const Params& p, int T, long long pages) {
  const bool pow2 = (p.g & (p.g - 1)) == 0;
  return T > 0 && pages > 0 && pow2 && p.g <= QROWS && p.page_size % 8 == 0 && p.page_size <= KT &&
         KT % p.page_size == 0 && ((uintptr_t)p.q % 16) == 0 && ((uintptr_t)p.k_pool % 16) == 0 &&
         ((uintptr_t)p.v_pool % 16) == 0 && ((uintptr_t)p.out % 16) == 0 && encode_fn() != nullptr;
}

int launch_tile_tc(const Params& p, int T, long long pages, int R, int max_q_len, cudaStream_t stream) {
  CUtensorMap qm, km, vm;
  const int tokens_per_tile = QROWS / p.g;
  // queries [T][Hq][head size] through boxes [tokens_per_tile][g][64]
  int rc = tensor_map(p.q, p.Hq, T, 0, p.g, tokens_per_tile, &qm);
  if (rc) return rc;
  // pools [pages][Hkv][page_size][head size] through boxes [1][1][page_size][64]
  rc = tensor_map(p.k_pool, p.page_size, p.Hkv, pages, p.page_size, 1, &km);
  if (rc) return rc;
  rc = tensor_map(p.v_pool, p.page_size, p.Hkv, pages, p.page_size, 1, &vm);
  if (rc) return rc;
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e = cudaFuncSetAttribute(attention_tile_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "attention_tc: %s", cudaGetErrorString(e));
    configured.done();
  }
  const int q_tiles = (max_q_len + tokens_per_tile - 1) / tokens_per_tile;
  const long long total = (long long)q_tiles * p.Hkv * R;
  if (total > 0x7fffffff) return gb::fail(GB_UNSUPPORTED, "attention_tc: %lld pieces of work", total);
  const int sms = tc_host::sm_count();
  dim3 grid((unsigned)(total < sms ? total : sms), 1, 1);
  return gb::check_pdl_launch(gb::launch_pdl(attention_tile_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream,
                                             dim3(1, 1, 1), qm, km, vm, p, q_tiles, (int)total),
                              "attention_tc (tile)");
}

int tile_tc_error_check() { return gb_err::fetch_and_clear(); }
int tile_tc_set_error_sink(int* host_word) { return gb_err::set_sink(host_word); }

}  // namespace attn

#else  // other head sizes: the mma.sync kernels

namespace attn {
bool tile_tc_takes(const Params&, int, long long) { return false; }
int launch_tile_tc(const Params&, int, long long, int, int, cudaStream_t) {
  return gb::fail(GB_UNSUPPORTED, "attention_tc: head size %d", GB_HEAD_DIM);
}
int tile_tc_error_check() { return 0; }
int tile_tc_set_error_sink(int*) { return 0; }
}  // namespace attn

#endif
