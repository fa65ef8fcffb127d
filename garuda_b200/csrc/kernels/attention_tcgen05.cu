// Causal grouped-query attention over the paged cache for prompt portions on the
// fifth-generation tensor cores: both matrix products of a tile are tcgen05.mma with
// accumulators in tensor memory, operands arrive by TMA, the softmax runs in 32-bit in
// registers between them.
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
//   warp 0   one lane: TMA. The query tile (a 3-D box [tokens][group][64], two buffers); per key
//            tile one 4-D box per page for keys and for values, four stages.
//   warp 1   one lane: S = Q K^T for the tile two ahead into one of two S buffers in tensor memory
//            (128 columns), then O_tile = P V of the tile whose softmax just ended into one of two O
//            buffers per group (64 columns each). V is read as it lies in the cache, keys along
//            the rows (an MN-major operand). This warp is the one the tensor cores wait for, so it
//            steps counters instead of dividing, advances descriptors made once, and learns the
//            pieces' lengths 32 at a time from its lanes.
//   warps 2-9  two groups of 128 threads; a thread owns a query row and its group's 64 keys of
//            every tile, an attention stream of its own: reads its 64 scores from tensor memory,
//            masks (only on tiles that touch a row's limits), running maximum, exp2 with the
//            scale folded in, writes P in bfloat16 into shared memory in the layout the second
//            product reads (128-byte swizzle), and adds the previous tile's O_tile, rescaled, to
//            its 64 sums in registers. At the end of a piece the two groups' streams are merged.
//            They also clear the value rows no query may read (a stray NaN times a zero
//            probability would spoil a sum).
// Measured on this hardware: a product with fewer than 128 columns costs as much as one with 128
// (about 70 cycles for M = 128, K = 16), which is why S is one 128-column product for both groups.
// Every wait is bounded; a wait that runs out sets the error word and the CTA winds down.
//
// Built for head size 64 only (one 128-byte swizzled row per key); other head sizes use the
// mma.sync kernels.
#include "attention_common.cuh"
#include "error_word.cuh"
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 64
#endif

#if GB_HEAD_DIM == 64

namespace {

using namespace tc;
using attn::Params;

constexpr int HD = 64;
constexpr int QROWS = 128;          // query rows per CTA
constexpr int KT = 128;             // keys per tile
constexpr int GROUPS = 2;           // softmax groups: each walks its own half of every key tile
constexpr int GK = KT / GROUPS;     // keys per group and tile
constexpr int STAGES = 4;
constexpr int ROW_BYTES = HD * 2;   // 128: one swizzled row
constexpr int Q_BYTES = QROWS * ROW_BYTES;
constexpr int K_BYTES = KT * ROW_BYTES, V_BYTES = K_BYTES;
constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
constexpr int P_BYTES = QROWS * GK * 2;             // one group's probabilities of a tile: [128 rows][128 bytes]
constexpr int SMEM_BYTES = 1024 + 2 * Q_BYTES + STAGES * STAGE_BYTES + GROUPS * 2 * P_BYTES;
constexpr int TMEM_COLS = 512;                      // S: 2 buffers x 2 groups x 64 columns; O: 2 groups x 2 buffers x 64
constexpr int O_COL0 = GROUPS * 2 * GK;
constexpr int THREADS = 64 + GROUPS * 128;
static_assert(GK == 64 && O_COL0 + GROUPS * 2 * HD <= TMEM_COLS, "tensor memory layout");


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
  __device__ __forceinline__ void next_tile(const Params& p) {
    if (++j >= w.n_tiles) next_item(p);
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
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full[2], q_empty[2], kv_full[STAGES], kv_empty[STAGES];
  __shared__ __align__(8) uint64_t s_ready[2], p_ready[GROUPS][2], o_ready[2];   // s and o: one for both groups (a commit costs the issuer about as much as a product)
  __shared__ float other_ml[QROWS][2];      // the second group's maximum and denominator, for the merge
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = tiles;                                      // two query buffers
  const uint32_t kv_s = tiles + 2 * Q_BYTES;                       // stage s: K at kv_s + s * STAGE_BYTES, V after it
  const uint32_t p_s = kv_s + STAGES * STAGE_BYTES;                // group g, buffer b at p_s + (2 g + b) * P_BYTES

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&q_full[b]), 1);
      mbar_init(smem_u32(&q_empty[b]), 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_ready[b]), 1);
      mbar_init(smem_u32(&o_ready[b]), 1);
      for (int g = 0; g < GROUPS; ++g) mbar_init(smem_u32(&p_ready[g][b]), 128);
    }
    abort_s = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&q_map);
    prefetch_tensormap(&k_map);
    prefetch_tensormap(&v_map);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  gb::pdl_launch_dependents();
  gb::pdl_wait();      // queries and this step's keys and values come from the kernel in front

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA
      const int page_shift = __ffs(p.page_size) - 1;         // pages are a power of two of keys
      const int pages_per_tile = KT >> page_shift;
      const uint32_t page_bytes = (uint32_t)p.page_size * ROW_BYTES;
      int gt = 0;               // tiles so far, over all items
      int stage = 0, par = 1;   // the stage to fill and the phase of its "empty" barrier to wait for
      Cursor c;
      for (c.start(p, q_tiles, total_items); !c.done; c.next_item(p)) {
        const Item& w = c.w;
        const int qb = c.it & 1;
        if (c.it >= 2 && !mbar_wait(smem_u32(&q_empty[qb]), ((c.it >> 1) & 1) ^ 1)) {
          gb_err::report(ERR_WAIT_EMPTY);
          abort_s = 1;
        }
        if (*(volatile int*)&abort_s) break;
        mbar_arrive_expect_tx(smem_u32(&q_full[qb]), Q_BYTES);
        tma_load_3d(q_s + qb * Q_BYTES, &q_map, smem_u32(&q_full[qb]), 0, w.kvh * p.g, w.q_begin + w.tok0);
        for (int j = 0; j < w.n_tiles; ++j, ++gt) {
          const int s = stage;
          const int key0 = (w.tile_begin + j) * KT;
          // pages that hold a key some row reads, and exist; looked up before waiting for the
          // stage, so that the table's latency passes during the wait
          int pages[16], count = 0;
          for (int g = 0; g < pages_per_tile; ++g) {
            const int first = key0 + g * p.page_size;
            pages[g] = (first <= w.hi && first + p.page_size > w.lo) ? w.table[first >> page_shift] : -1;
            count += pages[g] >= 0;
          }
          if (gt >= STAGES && !mbar_wait(smem_u32(&kv_empty[s]), par)) {
            gb_err::report(ERR_WAIT_EMPTY);
            abort_s = 1;
          }
          if (*(volatile int*)&abort_s) break;
          const uint32_t bar = smem_u32(&kv_full[s]);
          const uint32_t kdst = kv_s + s * STAGE_BYTES, vdst = kdst + K_BYTES;
          if (count == 0) {
            mbar_arrive(bar);
          } else {
            mbar_arrive_expect_tx(bar, 2u * count * page_bytes);
            for (int g = 0; g < pages_per_tile; ++g) {
              if (pages[g] < 0) continue;
              tma_load_4d(kdst + g * page_bytes, &k_map, bar, 0, 0, w.kvh, pages[g]);
              tma_load_4d(vdst + g * page_bytes, &v_map, bar, 0, 0, w.kvh, pages[g]);
            }
          }
          if (++stage == STAGES) stage = 0, par ^= 1;
        }
        if (*(volatile int*)&abort_s) break;
      }
      if (*(volatile int*)&abort_s) {
        // wind down: let the copies in flight land before the CTA's shared memory is given up
        for (int t = gt > STAGES ? gt - STAGES : 0; t < gt; ++t) {
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&kv_full[t % STAGES]), (t / STAGES) & 1)) {
            if (globaltimer_ns() - t0 > 20000000ull) {  // 20 ms
              gb_err::report(ERR_WAIT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    // The S products run two tiles ahead of the P V products, across the items' borders. Whatever
    // this warp executes between two products delays the tensor cores, so it is kept short: stage
    // and buffer counters are stepped, not divided; descriptors are made once and advanced. On
    // this hardware a product with fewer than 128 columns takes as long as one with 128 (about
    // 70 cycles for M = 128, K = 16), so S is computed for both groups at once (their S buffers
    // lie side by side). After a tile's softmax the S product two tiles ahead goes first: the
    // softmax warps wait for it next, for P V only a tile later.
    constexpr uint32_t idesc_s = instr_desc_bf16(QROWS, KT);
    constexpr uint32_t idesc_o = instr_desc_bf16(QROWS, HD) | INSTR_B_MN_MAJOR;
    const uint64_t dq0 = smem_desc_sw128(q_s), dk0 = smem_desc_sw128(kv_s), dv0 = smem_desc_sw128_mn(kv_s + K_BYTES),
                   dp0 = smem_desc_sw128(p_s);
    bool ok = true;
    TileWalk ws, wp;               // the S products' tile, the P V products' tile
    ws.start(p, q_tiles, total_items);
    wp = ws;
    int s_stage = 0, s_par = 0, p_stage = 0;       // stage (and its phase) of the S tile, stage of the P V tile
    int s_buf = 0;                                 // S buffer of the S tile
    int p_buf = 0, p_par = 0;                      // buffers of the P V tile and their phase
    auto issue_s = [&]() {      // S = Q K^T of the S tile into S buffer s_buf (both groups' columns)
      const int qb = ws.it & 1;
      if (ws.j == 0 && !mbar_wait(smem_u32(&q_full[qb]), (ws.it >> 1) & 1)) ok = false;
      if (ok && !mbar_wait(smem_u32(&kv_full[s_stage]), s_par)) ok = false;
      if (!ok) {
        if (lane == 0) gb_err::report(ERR_WAIT_FULL);
        return;
      }
      tc_fence_after_sync();
      if (lane == 0) {
        static_assert(HD / 16 == 4 && GK / 16 == 4, "four k steps per product");
        mma_bf16_x4(tmem_base + s_buf * KT, dq0 + (uint64_t)(qb * (Q_BYTES >> 4)),
                    dk0 + (uint64_t)(s_stage * (STAGE_BYTES >> 4)), idesc_s, 2, 2);
        mma_commit(smem_u32(&s_ready[s_buf]));
        if (ws.j == ws.n - 1) mma_commit(smem_u32(&q_empty[qb]));   // the item's queries have been read
      }
      __syncwarp();
      if (++s_stage == STAGES) s_stage = 0, s_par ^= 1;
      s_buf ^= 1;
      ws.next_tile(p, q_tiles, total_items);
    };
    if (!ws.done) issue_s();
    if (ok && !ws.done) issue_s();
    while (ok && !wp.done) {
      if (*(volatile int*)&abort_s) break;
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        if (ok && !mbar_wait(smem_u32(&p_ready[g][p_buf]), p_par)) {
          if (lane == 0) gb_err::report(ERR_WAIT_ACCUM);
          ok = false;
        }
      }
      if (!ok) break;
      // both groups have read this S buffer in full and written their P: first the S product that
      // takes the buffer over, then this tile's P V
      if (!ws.done) issue_s();
      if (!ok) break;
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
          mma_bf16_x4(tmem_base + O_COL0 + (2 * g + p_buf) * HD, dp0 + (uint64_t)((2 * g + p_buf) * (P_BYTES >> 4)),
                      dv0 + (uint64_t)(p_stage * (STAGE_BYTES >> 4) + g * (GK * ROW_BYTES >> 4)), idesc_o, 2,
                      16 * ROW_BYTES >> 4);
        }
        mma_commit(smem_u32(&o_ready[p_buf]));
        mma_commit(smem_u32(&kv_empty[p_stage]));     // keys and values of the stage have been read
      }
      __syncwarp();
      if (++p_stage == STAGES) p_stage = 0;
      p_par ^= p_buf;         // the phase flips after buffer 1
      p_buf ^= 1;
      wp.next_tile(p, q_tiles, total_items);
    }
    if (!ok) abort_s = 1;
  } else {
    // -------------------------------------------------------------------- softmax warps
    // Group g takes keys [g * 64, g * 64 + 64) of every tile: an attention stream of its own
    // (maximum, denominator, sums), merged with the other group's at the end. Two groups put two
    // warps on every scheduler, so that one computes while the other waits for tensor memory.
    const int grp = (warp - 2) >> 2;
    const int quarter = warp & 3;                        // the TMEM lanes this warp may read
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float scale_log2 = p.scale_log2;
    float* xo = reinterpret_cast<float*>(smem_raw + (p_s + 2 * P_BYTES - smem_u32(smem_raw)));
    bool ok = true;       // false: this thread only keeps the others company at the barriers
    int gt = 0;           // tiles so far, over all items
    int stage = 0;        // the current tile's stage of keys and values
    Cursor c;
    for (c.start(p, q_tiles, total_items); !c.done; c.next_item(p)) {
      const Item& w = c.w;
      const int row_pos = row < w.nrows ? w.pos0 + row / p.g : -1;       // no key is valid for a padding row
      const int row_start = (row < w.nrows && p.window > 0) ? max(0, row_pos + 1 - p.window) : 0;
      float o_acc[HD];
#pragma unroll
      for (int ch = 0; ch < HD; ++ch) o_acc[ch] = 0.f;
      float m = -INFINITY, l = 0.f, corr_saved = 0.f;      // m: running maximum of the raw dot products

      auto fold = [&](int t) {        // o_acc = o_acc * corr_saved + O_tile of the tile counted t
        if (!mbar_wait(smem_u32(&o_ready[t & 1]), (t >> 1) & 1)) {
          if (lane == 0) gb_err::report(ERR_WAIT_ACCUM);
          ok = false;
          abort_s = 1;
          return;
        }
        tc_fence_after_sync();
        uint32_t v[HD / 32][32];
#pragma unroll
        for (int h = 0; h < HD / 32; ++h) tmem_ld_32(lane_addr + O_COL0 + (2 * grp + (t & 1)) * HD + h * 32, v[h]);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < HD; ++ch) o_acc[ch] = fmaf(o_acc[ch], corr_saved, __uint_as_float(v[ch >> 5][ch & 31]));
      };

      for (int j = 0; j < w.n_tiles && ok; ++j, ++gt) {
        if (*(volatile int*)&abort_s) { ok = false; break; }
        if (!mbar_wait(smem_u32(&s_ready[gt & 1]), (gt >> 1) & 1)) {
          if (lane == 0) gb_err::report(ERR_WAIT_ACCUM);
          ok = false;
          abort_s = 1;
          break;
        }
        tc_fence_after_sync();
        {
          // Value rows that no row may read hold whatever was there (a page that was not fetched,
          // the unwritten end of the last page): their probabilities are zero, but zero times a
          // stray NaN is not. Clear them: half of each group's threads take one of the group's 64
          // rows each. (The stage has landed: S of this tile was computed from its keys. The
          // tensor core reads the values only after this thread's arrival below.)
          const int tile_key0 = (w.tile_begin + j) * KT;
          if ((tile_key0 < w.lo || tile_key0 + KT - 1 > w.hi) && row < GK) {
            const int vrow = grp * GK + row, key = tile_key0 + vrow;
            if (key < w.lo || key > w.hi) {
              const uint32_t vaddr = kv_s + stage * STAGE_BYTES + K_BYTES + vrow * ROW_BYTES;
#pragma unroll
              for (int ch = 0; ch < ROW_BYTES / 16; ++ch) st_shared_v4(vaddr + ch * 16, 0u, 0u, 0u, 0u);
            }
          }
          if (++stage == STAGES) stage = 0;
        }
        // the row's 64 scores of this group, one wait for the two loads
        uint32_t sv[GK / 32][32];
#pragma unroll
        for (int h = 0; h < GK / 32; ++h) tmem_ld_32(lane_addr + (2 * (gt & 1) + grp) * GK + h * 32, sv[h]);
        tmem_ld_wait();
        auto sc = [&](int ch) -> float& { return reinterpret_cast<float&>(sv[ch >> 5][ch & 31]); };
        const int key0 = (w.tile_begin + j) * KT + grp * GK;
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
        const float m_use = m_new == -INFINITY ? 0.f : m_new;          // nothing valid yet: avoid inf - inf
        const float corr = m == -INFINITY ? 0.f : fast_exp2((m - m_use) * scale_log2);
        const float neg_m = -m_use * scale_log2;
        m = m_new;
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t prow = p_s + (2 * grp + (gt & 1)) * P_BYTES + row * 128;
#pragma unroll
        for (int c8 = 0; c8 < GK / 8; ++c8) {
          float pr[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            pr[e] = fast_exp2(fmaf(sc(c8 * 8 + e), scale_log2, neg_m));   // exp2(-inf) = 0 for masked keys
            ls[e & 3] += pr[e];
          }
          // 16-byte chunk c8 of the row, swizzled with the row
          st_shared_v4(prow + ((c8 ^ (row & 7)) << 4), pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]),
                       pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
        }
        l = l * corr + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
        fence_proxy_async();            // the tensor core reads P through the async proxy
        tc_fence_before_sync();         // this thread's reads of S are over
        mbar_arrive(smem_u32(&p_ready[grp][gt & 1]));
        if (j > 0) fold(gt - 1);
        corr_saved = corr;
      }
      if (ok) fold(gt - 1);
      // ---- merge the two groups: the second hands its sums over through its own P buffers
      // (its last product has been read from them: fold waited for it), [channel][row] floats
      if (grp == 1 && ok) {
#pragma unroll
        for (int ch = 0; ch < HD; ++ch) xo[ch * QROWS + row] = o_acc[ch];
        other_ml[row][0] = m;
        other_ml[row][1] = l;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(GROUPS * 128) : "memory");
      if (grp == 0 && ok && row < w.nrows && !*(volatile int*)&abort_s) {
        const float m2 = other_ml[row][0], l2 = other_ml[row][1];
        const float mt = fmaxf(m, m2);
        const float f1 = m == -INFINITY ? 0.f : fast_exp2((m - mt) * scale_log2);
        const float f2 = m2 == -INFINITY ? 0.f : fast_exp2((m2 - mt) * scale_log2);
        const float lt = l * f1 + l2 * f2;
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
        const float a1 = f1 * inv, a2 = f2 * inv;
        __nv_bfloat16* dst = p.out + ((size_t)(w.q_begin + w.tok0 + row / p.g) * p.Hq + w.kvh * p.g + row % p.g) * HD;
#pragma unroll
        for (int ch = 0; ch < HD; ch += 8) {
          float t[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) t[e] = o_acc[ch + e] * a1 + xo[(ch + e) * QROWS + row] * a2;
          uint4 wv;
          wv.x = pack_bf16(t[0], t[1]);
          wv.y = pack_bf16(t[2], t[3]);
          wv.z = pack_bf16(t[4], t[5]);
          wv.w = pack_bf16(t[6], t[7]);
          *reinterpret_cast<uint4*>(dst + ch) = wv;
        }
      }
      // the second group's next probabilities go where its sums were just read
      asm volatile("bar.sync 1, %0;" ::"n"(GROUPS * 128) : "memory");
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
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

// A bf16 tensor [d3][d2][d1][64] (64 contiguous) seen through boxes [1][b2][b1][64] (d3 = 0: three
// dimensions, box [b2][b1][64]), 128-byte swizzle; elements outside read as zeros.
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
  cuuint32_t box[4] = {(cuuint32_t)HD, (cuuint32_t)b1, (cuuint32_t)b2, 1};
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
  // queries [T][Hq][64] through boxes [tokens_per_tile][g][64]
  int rc = tensor_map(p.q, p.Hq, T, 0, p.g, tokens_per_tile, &qm);
  if (rc) return rc;
  // pools [pages][Hkv][page_size][64] through boxes [1][1][page_size][64]
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
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
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
