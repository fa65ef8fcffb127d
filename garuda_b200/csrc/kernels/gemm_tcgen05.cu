// bfloat16 matrix products on the 5th-generation tensor cores:
//   out[Mx, Nw] (+)= x[Mx, K] * w[Nw, K]^T        (garuda/src/simd/mod.rs:96-129)
// and the fused gate/up product with the SiLU-gate of the feed-forward
//   out[Mx, F] = silu(x * gate^T) * (x * up^T)     (garuda/src/llama/mod.rs:1013-1017)
// for which gate and up rows are packed into one matrix in groups of 64: rows
// [128 g, 128 g + 64) are gate rows 64 g .., the next 64 the matching up rows
// (zero rows pad the last group), so that every 128-row tile holds the gate and
// the up values of the same 64 output features.
//
// One CTA computes a 128 x BN tile: a producer thread streams 128x64 and BNx64
// operand tiles into shared memory with TMA (128-byte swizzle), one thread
// issues tcgen05.mma with the accumulator in tensor memory, and when the last
// MMA has retired the four warps read the accumulator back with tcgen05.ld and
// run the epilogue. Accumulation is 32-bit.
//
// Two orientations. With many tokens the 128 rows of the MMA are tokens and the
// BN columns are output features. With few tokens (decode) the operands swap:
// the 128 MMA rows are output features (weight rows) and the BN = 16..64 columns
// are tokens, so that the weight stream fills the tensor core's rows and the
// result is written transposed.
//
// In the swapped orientation a matrix has few 128-row tiles (16 to 44 for a
// 2048-wide layer), too few CTAs to pull memory at full rate. There the K range
// is split over the CTAs of a thread-block cluster: every CTA accumulates its
// share of K in its own tensor memory, the others send their partial sums into
// the leader's shared memory (distributed shared memory), and the leader adds
// them in rank order and runs the epilogue. No scratch in global memory, no
// atomics, and the same sum order every time.
//
// An RMS norm that stands between two products is folded into them (EpilogueArgs):
// the product in front, which adds into the residual stream x, also writes
// x * weight in bfloat16 and per-token partial sums of x^2; the product behind
// takes those rows as its tokens and multiplies its results by
// 1/sqrt(mean(x^2) + eps). No norm kernel, and no second pass over x.
//
// Rows outside a matrix are zero-filled by TMA and masked in the epilogue; K
// need not be a multiple of 64 (the tail is zero-filled) but must be a multiple
// of 8, because a TMA row pitch is a multiple of 16 bytes.
#include "error_word.cuh"
#include "tc_common.cuh"
#include "tc_host.cuh"

namespace {

using namespace tc;
using namespace tc_host;

constexpr int BM = 128;   // MMA rows per CTA
constexpr int BK = 64;    // bf16 per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int SMEM_LIMIT = 227 * 1024;          // most dynamic shared memory a CTA can have
constexpr int SMEM_BUDGET_LARGE = 200 * 1024;   // many tokens: one CTA per SM, all of it pipeline
constexpr int SMEM_BUDGET_SMALL = 110 * 1024;   // up to 16 tokens: pipeline depth that the stream of weights needs
// 32 or 64 tokens: a CTA has 20 or 24 KB per step of K in flight, and what is in flight bounds what
// it takes in (four stages of 24 KB against 2 us of latency are 48 GB/s): as deep as fits
constexpr int SMEM_BUDGET_MID = 192 * 1024;
constexpr int SMEM_BUDGET_DUAL = 140 * 1024;    // few tokens, gate and up together

// EPI_ACCUMULATE_NORM: accumulate, and fold in the first half of the norm that follows (EpilogueArgs::h_out);
// chosen by the host, a variant of its own so that the plain accumulation's code stays as it is
enum Epilogue : int { EPI_STORE = 0, EPI_ACCUMULATE = 1, EPI_SWIGLU = 2, EPI_ROPE = 3, EPI_ACCUMULATE_NORM = 4 };

// What the epilogues need beyond the output pointer. For the query/key/value epilogue: the output features are (heads + 2 kv_heads) heads of
// head_dim; query and key heads are rotated at the token's position (garuda/src/simd/mod.rs:196-206,
// angle = (float)pos * inv_freq[i] in 32-bit; the cosines and sines are made once per step for all
// layers by rope_table in elementwise.cu), queries go to q_out, rotated keys and raw values into
// their pages (garuda/src/llama/mod.rs:784-791). head_dim divides 128, so no head straddles a tile.
struct EpilogueArgs {
  __nv_bfloat16* q_out;          // [T, heads, head_dim]
  __nv_bfloat16* k_pool;         // [pages, kv_heads, page_size, head_dim]
  __nv_bfloat16* v_pool;
  const int32_t* positions;      // [T]
  const int32_t* token_req;      // [T]
  const int32_t* block_table;    // [R, table_width]
  const float2* cs;              // [T, head_dim / 2] (cos, sin) of every token's angles, or null: no rotation
  int table_width, heads, kv_heads, head_dim, interleaved, page_size;
  // An RMS norm folded into the two products around it (garuda/src/simd/mod.rs:166-173,
  // garuda/src/llama/mod.rs:733-738). The product in front, which adds into the residual stream,
  // also writes x * weight in bfloat16 (x: the new residual value) and, per tile of 128 features,
  // the sum of x^2 over the tile for every token. The product behind reads those rows as its
  // tokens and multiplies its results by 1/sqrt(sum x^2 / width + eps) of their token, which gives
  // (x * rms * weight) W^T with the sum, the root and the scaling in 32-bit.
  const float* sums_in;          // consumer: [tiles_in, sums_ld] partial sums of squares, or null
  int tiles_in;
  float eps, inv_width;
  __nv_bfloat16* h_out;          // producer: [T, features] x * weight, or null
  const float* weight;           // [features]
  float* sums_out;               // [tiles of 128 features, sums_ld]
  int sums_ld;                   // tokens
  // The weights that the kernel after this one will stream (or null): while this kernel waits out its
  // chain of latencies (activations, products, reduction, epilogue) the memory system is idle, so its
  // CTAs ask for those weights to be brought into L2 meanwhile, each a slice.
  const uint8_t* next_stream;
  long long next_bytes;
};

// This CTA's slice of `bytes` at `base` into L2 (cta of ctas; 16-byte granules), by one thread.
__device__ __forceinline__ void prefetch_slice_l2(const uint8_t* base, long long bytes, int cta, int ctas) {
  if (base == nullptr || bytes <= 0) return;
  const long long granules = bytes >> 4;
  const long long per = (granules + ctas - 1) / ctas;
  long long begin = per * cta, end = begin + per;
  if (end > granules) end = granules;
  constexpr long long CHUNK = 4096;        // granules per instruction: 64 KB
  for (long long g = begin; g < end; g += CHUNK) {
    const uint32_t size = (uint32_t)(((end - g) < CHUNK ? (end - g) : CHUNK) << 4);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + (g << 4)), "r"(size) : "memory");
  }
}

// Where feature `head`, channel d of the token at `pos` (request row `req`) is stored; null if the
// position has no page.
__device__ __forceinline__ __nv_bfloat16* rope_destination(const EpilogueArgs& ra, int token, int req, int pos,
                                                           int head, int d) {
  if (head < ra.heads) return ra.q_out + ((size_t)token * ra.heads + head) * ra.head_dim + d;
  const int page = ra.block_table[(size_t)req * ra.table_width + pos / ra.page_size];
  if (page < 0) return nullptr;
  const bool is_k = head < ra.heads + ra.kv_heads;
  const int kvh = head - ra.heads - (is_k ? 0 : ra.kv_heads);
  return (is_k ? ra.k_pool : ra.v_pool) +
         (((size_t)page * ra.kv_heads + kvh) * ra.page_size + pos % ra.page_size) * ra.head_dim + d;
}


// Bytes of the rotation's tables in the few-token kernel: cosines and sines [BN tokens][64
// frequencies] and each token's row in the pools.
__host__ __device__ constexpr int rope_table_bytes(int epi, int bn) { return epi == EPI_ROPE ? bn * 64 * 8 + bn * 8 : 0; }

template <int BN, bool DUAL_M, bool DUAL_N, bool TRANS = false, int EXTRA = 0>
struct Geometry {
  static constexpr int NUM_M = DUAL_M ? 2 : 1, NUM_N = DUAL_N ? 2 : 1;
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = NUM_M * A_BYTES + NUM_N * B_BYTES;
  // shared memory for the operand pipeline; the swapped orientation leaves room for the partial sums
  // that the other CTAs of a cluster send, and (without them) for a second CTA on the SM
  static constexpr int PIPE_BUDGET = !TRANS ? SMEM_BUDGET_LARGE
                                     : DUAL_M ? SMEM_BUDGET_DUAL : BN >= 32 ? SMEM_BUDGET_MID : SMEM_BUDGET_SMALL;
  static constexpr int STAGES = (PIPE_BUDGET / STAGE_BYTES) < 8 ? (PIPE_BUDGET / STAGE_BYTES) : 8;
  static constexpr int ACCUMULATORS = NUM_M * NUM_N;
  static constexpr int COLS_NEEDED = ACCUMULATORS * BN;
  static constexpr int TMEM_COLS = COLS_NEEDED <= 32 ? 32 : COLS_NEEDED <= 64 ? 64 : COLS_NEEDED <= 128 ? 128
                                   : COLS_NEEDED <= 256 ? 256 : 512;
  static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;
  // The CTAs of a cluster exchange partial sums in chunks of 16 columns (tokens): chunk c is summed
  // and written out by rank c % owners, owners = min(cluster, chunks); every other rank sends it
  // its 16 columns of that chunk. A rank thus receives (cluster - 1) x (its chunks) x 8 KB.
  static constexpr int CHUNKS = ACCUMULATORS * BN / 16;
  static constexpr int CHUNK_BYTES = 16 * BM * 4;
  static constexpr int owners(int cluster) { return cluster < CHUNKS ? cluster : CHUNKS; }
  static constexpr int owned_most(int cluster) { return (CHUNKS + owners(cluster) - 1) / owners(cluster); }
  static constexpr int receive_bytes(int cluster) { return (cluster - 1) * owned_most(cluster) * CHUNK_BYTES; }
  // statically declared shared memory (barriers) comes out of the same limit; EXTRA bytes lie
  // between the pipeline and the partial sums
  static constexpr int STATIC_RESERVE = 2 * 1024;
  // + slack to align the tiles to 1024 B
  static constexpr int smem_bytes(int cluster, int stages = STAGES) {
    return stages * STAGE_BYTES + 1024 + EXTRA + receive_bytes(cluster);
  }
  // the most stages (at most STAGES) with which a cluster of this size fits; 0: it does not fit
  static constexpr int stages_that_fit(int cluster) {
    int st = STAGES;
    while (st >= 2 && smem_bytes(cluster, st) + STATIC_RESERVE > SMEM_LIMIT) --st;
    return st >= 2 ? st : 0;
  }
  static constexpr int max_cluster() {
    int best = 1;
    for (int c = 2; c <= 8; ++c)
      if (stages_that_fit(c) >= (STAGES < 4 ? STAGES : 4)) best = c;
    return best;
  }
  static constexpr int MAX_CLUSTER = !TRANS ? 1 : max_cluster();
  static constexpr int most_smem() {      // over the cluster sizes that fit
    int most = smem_bytes(1, stages_that_fit(1));
    for (int c = 2; c <= 8; ++c)
      if (stages_that_fit(c) > 0 && smem_bytes(c, stages_that_fit(c)) > most) most = smem_bytes(c, stages_that_fit(c));
    return most;
  }
  static_assert(2 * STAGE_BYTES + 1024 + EXTRA + STATIC_RESERVE <= SMEM_LIMIT, "tile and tables too large for shared memory");
  static constexpr int SMEM_BYTES = smem_bytes(1);
  static_assert(STAGES >= 2, "tile too large for shared memory");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M = 128");
};

template <typename OT>
__device__ __forceinline__ void store_value(OT* p, float v);
template <>
__device__ __forceinline__ void store_value<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_value<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// The SiLU-gate of the fused epilogues. The exponential is the hardware's fast one: its error
// (about 2 ulp of a float) is far below the rounding of the bfloat16 result.
__device__ __forceinline__ float silu_gate_fast(float g, float u) {
  return g * __frcp_rn(1.0f + __expf(-g)) * u;
}

// Sums each of sixteen values over the lanes of a warp with sixteen shuffles: at every step a
// lane keeps half of its values and hands the other half to its partner, which keeps those. Lane
// L ends with the sum of value warp_sum16_index(L) (lanes 2k and 2k + 1 hold the same). The order
// of the additions is fixed.
__device__ __forceinline__ int warp_sum16_index(int lane) {
  return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
}
__device__ __forceinline__ float warp_sum16(const float (&v)[16], int lane) {
  float a8[8], a4[4], a2[2];
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    a8[i] = (b4 ? v[i + 8] : v[i]) + __shfl_xor_sync(0xffffffffu, b4 ? v[i] : v[i + 8], 16);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    a4[i] = (b3 ? a8[i + 4] : a8[i]) + __shfl_xor_sync(0xffffffffu, b3 ? a8[i] : a8[i + 4], 8);
#pragma unroll
  for (int i = 0; i < 2; ++i)
    a2[i] = (b2 ? a4[i + 2] : a4[i]) + __shfl_xor_sync(0xffffffffu, b2 ? a4[i] : a4[i + 2], 4);
  const float a1 = (b1 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, b1 ? a2[0] : a2[1], 2);
  return a1 + __shfl_xor_sync(0xffffffffu, a1, 1);
}

constexpr int C_THREADS = 192;   // warp 0: producer, warp 1: MMA issuer, warps 2-5: epilogue

// Few tokens. rows_m / rows_n: valid rows of the MMA-row operand (the weights: output features)
// and of the MMA-column operand (the tokens). The output is written transposed: out[token][feature].
// The CTAs of a cluster (gridDim.z of them, along z) split the K blocks, kb_per_rank each. The
// tile's columns (tokens) are shared out in chunks of 16 among the first ranks (with 16 tokens:
// rank 0 alone): a rank sends every chunk that is not its own to the chunk's owner with st.async,
// counted on the owner's mbarrier; the owner adds the ranks' sums in rank order and writes the
// chunk out. With 32 or 64 tokens the exchange, the epilogue and the memory for what is received
// are thus spread over up to four CTAs.
template <int BN, int EPI, typename OT>
__global__ void __launch_bounds__(C_THREADS, 1)
gemm_tc_cluster_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_n,
                       OT* __restrict__ out, int ldo, int rows_m, int rows_n, int K, int kb_per_rank,
                       const EpilogueArgs ra, const int stages) {
  constexpr bool DUAL_M = false;
  using G = Geometry<BN, false, false, true, rope_table_bytes(EPI, BN)>;
  constexpr int STAGES = G::STAGES;          // the most; `stages` of them are used (fewer: two CTAs fit on an SM)
  constexpr int ACC = G::ACCUMULATORS;
  // With so few columns an MMA is over long before the next one that adds to the same accumulator
  // may start. The four MMAs of a K block therefore go to four accumulators of their own (four
  // independent chains); the epilogue adds the four.
  constexpr int KSPLIT = BK / UMMA_K;
  constexpr int ACC_COLS = ACC * BN;                     // columns of one of the four
  constexpr int TMEM_COLS = KSPLIT * ACC_COLS <= 32 ? 32 : KSPLIT * ACC_COLS <= 64 ? 64
                            : KSPLIT * ACC_COLS <= 128 ? 128 : KSPLIT * ACC_COLS <= 256 ? 256 : 512;
  static_assert(KSPLIT * ACC_COLS <= 512, "accumulators exceed tensor memory");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t accum_bar;
  __shared__ __align__(8) uint64_t partial_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ float inv_s[BN];       // folded norm: 1/rms of this tile's tokens

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int total_kb = (K + BK - 1) / BK;
  const int rank = (int)blockIdx.z, ranks = (int)gridDim.z;
  const int kb_begin = rank * kb_per_rank;
  const int num_kb = max(min(total_kb, kb_begin + kb_per_rank) - kb_begin, 0);
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // what a rank receives: [sender, in rank order without itself][its chunk][16 columns][128 rows]
  // floats: the threads of a warp (consecutive rows) write and read consecutive words, so neither
  // the remote stores nor the owner's loads collide on a bank
  const uint32_t pipe_bytes = (uint32_t)stages * G::STAGE_BYTES;
  const uint32_t partials = tiles + pipe_bytes + rope_table_bytes(EPI, BN);
  // chunk c of 16 tokens belongs to rank c % owners; this rank's are rank, rank + owners, ...
  constexpr int CHUNKS = G::CHUNKS;
  const int owners = ranks < CHUNKS ? ranks : CHUNKS;
  const int owned_most = (CHUNKS + owners - 1) / owners;
  const int my_chunks = rank < owners ? (CHUNKS - rank + owners - 1) / owners : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&accum_bar), 1);
    mbar_init(smem_u32(&partial_bar), 1);
    abort_s = 0;
    fence_barrier_init();
    if (my_chunks > 0 && ranks > 1)
      mbar_arrive_expect_tx(smem_u32(&partial_bar), (uint32_t)((ranks - 1) * my_chunks * G::CHUNK_BYTES));
    fence_proxy_async();
    prefetch_tensormap(&map_m);
    prefetch_tensormap(&map_n);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  // Rank 0's barrier is armed before anyone may send to it. This is the only cluster-wide
  // barrier, and it is passed while the kernel in front is still running.
  if (ranks > 1) cluster_arrive_wait();
  gb::pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // -------------------------------------------------------------- producer
      // The weights are written by no kernel: their first tiles are fetched before waiting for
      // the kernel in front; the tokens' tiles after.
      int issued = 0;
      const int early = min(stages, num_kb);
      for (int it = 0; it < early; ++it) {
        const uint32_t bar = smem_u32(&full_bar[it]);
        const uint32_t base = tiles + it * G::STAGE_BYTES;
        const int k0 = (kb_begin + it) * BK;
        mbar_arrive_expect_tx(bar, G::STAGE_BYTES);
        tma_load_2d(base, &map_m, bar, k0, m0);
      }
      gb::pdl_wait();
      for (int it = 0; it < early; ++it) {
        tma_load_2d(tiles + it * G::STAGE_BYTES + G::NUM_M * G::A_BYTES, &map_n, smem_u32(&full_bar[it]),
                    (kb_begin + it) * BK, n0);
        issued = it + 1;
      }
      // the first `early` blocks filled stages 0 .. early - 1 in their first phase
      int s = early == stages ? 0 : early, par = early == stages ? 0 : 1;
      for (int it = early; it < num_kb; ++it, s = (s + 1 == stages ? 0 : s + 1), par ^= (s == 0)) {
        if (!mbar_wait(smem_u32(&empty_bar[s]), par)) {
          gb_err::report(ERR_WAIT_EMPTY);
          abort_s = 1;
        }
        if (*(volatile int*)&abort_s) break;
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t base = tiles + s * G::STAGE_BYTES;
        const int k0 = (kb_begin + it) * BK;
        mbar_arrive_expect_tx(bar, G::STAGE_BYTES);
        tma_load_2d(base, &map_m, bar, k0, m0);
        tma_load_2d(base + G::NUM_M * G::A_BYTES, &map_n, bar, k0, n0);
        issued = it + 1;
      }
      // everything of this CTA's own stream has been asked for: now the next kernel's weights
      prefetch_slice_l2(ra.next_stream, ra.next_bytes,
                        (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)),
                        (int)(gridDim.x * gridDim.y * gridDim.z));
      if (*(volatile int*)&abort_s) {
        // wind down: let the copies already in flight land before the CTA's shared memory is given up
        for (int it = issued > stages ? issued - stages : 0; it < issued; ++it) {
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&full_bar[it % stages]), (it / stages) & 1)) {
            if (globaltimer_ns() - t0 > 20000000ull) {  // 20 ms
              gb_err::report(ERR_WAIT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // -------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
      int s = 0, par = 0;
      for (int it = 0; it < num_kb; ++it, s = (s + 1 == stages ? 0 : s + 1), par ^= (s == 0)) {
        if (!mbar_wait(smem_u32(&full_bar[s]), par)) {
          gb_err::report(ERR_WAIT_FULL);
          abort_s = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t base = tiles + s * G::STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t koff = k * UMMA_K * 2;  // bytes along the swizzled row
          const bool acc = it > 0;
          const uint32_t d = tmem_base + k * ACC_COLS;
          const uint64_t db = smem_desc_sw128(base + G::NUM_M * G::A_BYTES + koff);
          mma_bf16(d, smem_desc_sw128(base + koff), db, idesc, acc);
        }
        mma_commit(smem_u32(&empty_bar[s]));  // the stage is free once these MMAs have read it
      }
      mma_commit(smem_u32(&accum_bar));       // fires when every MMA above has retired
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;                         // the TMEM lanes this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const int row = m0 + row_in_tile;                     // output feature
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    // Rotation: the epilogue threads of the leading CTA fill, before anything else,
    // a table of cosines and sines [token][frequency] and each token's row in the pools, sharing
    // the work (a thread alone would compute every angle of its feature: thousands of dependent
    // instructions). Positions, request rows and block tables are written by copies that end
    // before the first kernel of a chain starts, so they are read without waiting for the kernel
    // in front. The table is complete for every thread after the first barrier of the loop below.
    constexpr bool ROPE_EARLY = EPI == EPI_ROPE;
    float (*rope_cs)[64] = reinterpret_cast<float (*)[64]>(smem_raw + (tiles - smem_u32(smem_raw)) + pipe_bytes);
    float (*rope_sn)[64] = rope_cs + BN;
    long long* rope_slot = reinterpret_cast<long long*>(rope_sn + BN);   // element offset of the token's row, head 0; -1: no page
    if (ROPE_EARLY && my_chunks > 0) {
      const int t = (int)threadIdx.x - 64;
      const int half = ra.head_dim >> 1, lg = 31 - __clz(half);      // head_dim divides 128: a power of two
      // only the tokens of this rank's chunks (with 64 tokens and heads of 128 the whole table is
      // 4,096 entries, 32 loads in a row for every thread, and took longer than the product)
      for (int q = 0; q < my_chunks; ++q) {
        const int c = (rank + q * owners) * 16;
#pragma unroll 4
        for (int e = t; e < 16 * half; e += 128) {
          const int j = c + (e >> lg), fi = e & (half - 1);
          float sn = 0.f, cs = 1.f;
          if (ra.cs != nullptr && n0 + j < rows_n) {
            const float2 v = ra.cs[(size_t)(n0 + j) * half + fi];
            cs = v.x, sn = v.y;
          }
          rope_cs[j][fi] = cs;
          rope_sn[j][fi] = sn;
        }
      }
      if (t < BN) {
        long long slot = -1;
        const int col = n0 + t;
        if (col < rows_n && ra.kv_heads > 0) {
          const int pos = ra.positions[col];
          const int page = ra.block_table[(size_t)ra.token_req[col] * ra.table_width + pos / ra.page_size];
          if (page >= 0) slot = (((long long)page * ra.kv_heads) * ra.page_size + pos % ra.page_size) * ra.head_dim;
        }
        rope_slot[t] = slot;
      }
    }
    constexpr bool emit = EPI == EPI_ACCUMULATE_NORM;                    // the norm behind this product is folded in
    constexpr bool ADD = EPI == EPI_ACCUMULATE || emit;
    float old[ADD ? BN : 1];                 // of this rank's chunks, in their order
    // each epilogue warp's sum of squares per token, in the pipeline's memory (idle by then; static
    // shared memory is kept small, so that two CTAs still fit on an SM)
    float (*red_s)[BN] = reinterpret_cast<float (*)[BN]>(smem_raw + (tiles - smem_u32(smem_raw)));
    float w_row = 0.f;
    if (my_chunks > 0) {
      if (emit && row < rows_m) w_row = ra.weight[row];                 // a model constant: no need to wait
      gb::pdl_wait();
      if (ADD) {
        // what is to be added to is fetched while the matrix product runs
#pragma unroll
        for (int q = 0; q < CHUNKS; ++q) {
          const int c = (rank + q * owners) * 16;       // first column of this rank's q-th chunk
#pragma unroll
          for (int j = 0; j < 16; ++j)
            old[ADD ? q * 16 + j : 0] = (q < my_chunks && row < rows_m && n0 + c + j < rows_n)
                                            ? gb::to_float<OT>(out[(size_t)(n0 + c + j) * ldo + row]) : 0.f;
        }
      }
      if (ra.sums_in != nullptr) {
        // the norm in front of this product: 1/rms of every token, from the partial sums (in tile
        // order: the same sum whatever else is in the batch)
        const int t = (int)threadIdx.x - 64;
        if (t < BN) {
          float s = 0.f;
          if (n0 + t < rows_n)
            for (int i = 0; i < ra.tiles_in; ++i) s += ra.sums_in[(size_t)i * ra.sums_ld + n0 + t];
          inv_s[t] = rsqrtf(s * ra.inv_width + ra.eps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
    bool have = mbar_wait(smem_u32(&accum_bar), 0);
    if (!have && lane == 0) gb_err::report(ERR_WAIT_ACCUM);
    have = have && !*(volatile int*)&abort_s;
    tc_fence_after_sync();

    // 16 columns of this thread's row, summed over the four accumulators
    auto load16 = [&](int col, float (&v)[16]) {
      uint32_t r[KSPLIT][16];
#pragma unroll
      for (int q = 0; q < KSPLIT; ++q) tmem_ld_16(taddr + q * ACC_COLS + col, r[q]);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float t = __uint_as_float(r[0][j]);
#pragma unroll
        for (int q = 1; q < KSPLIT; ++q) t += __uint_as_float(r[q][j]);
        v[j] = t;
      }
    };

    if (ranks > 1 && num_kb > 0) {
      // this thread's row of every chunk that another rank owns, into that rank's shared memory
      const int slot_of_mine = rank;         // among the senders of an owner o: rank if rank < o, else rank - 1
#pragma unroll 1
      for (int ch = 0; ch < CHUNKS; ++ch) {
        const int o = ch % owners;
        if (o == rank) continue;
        const int slot = slot_of_mine < o ? slot_of_mine : slot_of_mine - 1;
        const uint32_t there = partials + (uint32_t)((slot * owned_most + ch / owners) * G::CHUNK_BYTES) + (uint32_t)row_in_tile * 4;
        const uint32_t remote = map_to_rank(there, (uint32_t)o);
        const uint32_t remote_bar = map_to_rank(smem_u32(&partial_bar), (uint32_t)o);
        float v[16];
        load16(ch * 16, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) st_async_f32(remote + (uint32_t)j * (BM * 4), remote_bar, have ? v[j] : 0.f);
      }
    }
    if (my_chunks > 0) {
      if (ranks > 1) {
        const bool got = mbar_wait(smem_u32(&partial_bar), 0);
        if (!got && lane == 0) gb_err::report(ERR_WAIT_ACCUM);
        have = have && got;
      }
      if (have) {
        const float* partial = reinterpret_cast<const float*>(smem_raw + (partials - smem_u32(smem_raw))) +
                               row_in_tile;
        // SiLU-gate: rows 0-63 of the tile are gate rows, rows 64-127 the up rows of the same 64
        // features. The up half hands its values over through shared memory (the pipeline's, which
        // is idle by now).
        float* xch = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)));   // [16][64 or 128]
#pragma unroll
        for (int q = 0; q < CHUNKS; ++q) {
          if (q >= my_chunks) break;
          const int c = (rank + q * owners) * 16;       // first column of this rank's q-th chunk
          float own[16], v[16];
          load16(c, own);
          // all ranks' sums in rank order (the same sum every time), this rank's own in its place;
          // sixteen independent loads per rank, so that they overlap
          if (CHUNKS == 1) {        // rank 0 owns the one chunk
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = own[j];
            for (int pr = 1; pr < ranks; ++pr) {
              const float* src = partial + (size_t)(pr - 1) * (G::CHUNK_BYTES / 4);
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += src[j * BM];
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
            for (int pr = 0; pr < ranks; ++pr) {
              if (pr == rank) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += own[j];
              } else {
                const float* src = partial + (size_t)(((pr < rank ? pr : pr - 1) * owned_most + q) * (G::CHUNK_BYTES / 4));
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += src[j * BM];
              }
            }
          }
          if (ra.sums_in != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= inv_s[c + j];
          }
          if (EPI == EPI_SWIGLU) {
            if (row_in_tile >= 64) {
#pragma unroll
              for (int j = 0; j < 16; ++j) xch[j * 64 + row_in_tile - 64] = v[j];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
            const int feature = (m0 >> 1) + row_in_tile;         // 64 features per 128-row tile
            if (row_in_tile < 64 && feature < rows_m) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int col = n0 + c + j;      // token
                if (col < rows_n)
                  store_value<OT>(out + (size_t)col * ldo + feature, silu_gate_fast(v[j], xch[j * 64 + row_in_tile]));
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");      // before the next chunk reuses the buffer
          } else if (EPI == EPI_ROPE) {
            // A rotation pairs two rows of the tile (channels i and i + head_dim / 2 of a head, or
            // 2i and 2i + 1): every thread shows its values, then computes its own rotated channel.
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[j * BM + row_in_tile] = v[j];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (row < rows_m) {
              const int hd = ra.head_dim, half = hd >> 1;
              const int head = row / hd, d = row % hd;
              const bool rotate = ra.cs != nullptr && head < ra.heads + ra.kv_heads;
              const bool low = ra.interleaved ? (d & 1) == 0 : d < half;
              const int partner = ra.interleaved ? (row_in_tile ^ 1) : (low ? row_in_tile + half : row_in_tile - half);
              if (ROPE_EARLY) {
                const int fi = ra.interleaved ? d >> 1 : d & (half - 1);
                const bool is_q = head < ra.heads, is_k = head < ra.heads + ra.kv_heads;
                __nv_bfloat16* base = is_q ? ra.q_out + row
                                           : (is_k ? ra.k_pool : ra.v_pool) +
                                                 (size_t)(head - ra.heads - (is_k ? 0 : ra.kv_heads)) * ra.page_size * hd + d;
                const size_t q_stride = (size_t)ra.heads * hd;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const int e = ROPE_EARLY ? c + j : 0;
                  const int col = n0 + c + j;
                  const float other = xch[j * BM + partner];
                  const float cs = rope_cs[e][fi], sn = rope_sn[e][fi];
                  const float x = !rotate ? v[j] : low ? v[j] * cs - other * sn : other * sn + v[j] * cs;
                  const long long slot = rope_slot[e];
                  if (col < rows_n && (is_q || slot >= 0))
                    base[is_q ? (size_t)col * q_stride : (size_t)slot] = __float2bfloat16_rn(x);
                }
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          } else {
            float sq[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = n0 + c + j;      // token
              sq[j] = 0.f;
              if (row >= rows_m || col >= rows_n) continue;
              float x = v[j];
              if (ADD) x += old[ADD ? q * 16 + j : 0];
              store_value<OT>(out + (size_t)col * ldo + row, x);
              if (emit) {
                ra.h_out[(size_t)col * ldo + row] = __float2bfloat16_rn(x * w_row);
                sq[j] = x * x;
              }
            }
            if (emit) {
              const float total = warp_sum16(sq, lane);
              if ((lane & 1) == 0) red_s[quarter][c + warp_sum16_index(lane)] = total;
            }
          }
        }
        if (emit) {
          // this tile's sum of squares for every token: the four warps' parts in a fixed order
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int t = (int)threadIdx.x - 64;
          if (t < BN && (t >> 4) % owners == rank && n0 + t < rows_n)      // the tokens of this rank's chunks
            ra.sums_out[(size_t)blockIdx.y * ra.sums_ld + n0 + t] = red_s[0][t] + red_s[1][t] + red_s[2][t] + red_s[3][t];
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// --------------------------------------------------------------------------
// Many tokens: a persistent kernel. One CTA per SM walks a list of 128 x BN
// tiles. Warp 0 feeds the shared-memory pipeline, warp 1 issues the MMAs into
// one of two accumulator stages in tensor memory, warps 2-5 drain the other
// stage (tcgen05.ld, epilogue arithmetic, 16-byte stores), so the epilogue of a
// tile runs under the matrix product of the next.
// Epilogue warps of the many-token kernels: two per lane quarter, each with half of a tile's columns
// (twice the loads and stores in flight), except for the rotation's epilogue, whose threads need
// whole heads and many registers.
__host__ __device__ constexpr int epilogue_warps(int epi) { return epi == EPI_ROPE ? 4 : 8; }
__host__ __device__ constexpr int p_threads(int epi) { return 64 + 32 * epilogue_warps(epi); }
// The columns [begin, end) of a BN-wide tile for the first or second warp of a quarter.
__device__ __forceinline__ void epilogue_columns(int epi, int bn, int which, int& begin, int& end) {
  const int unit = epi == EPI_SWIGLU ? 128 : 32;
  const int mid = epilogue_warps(epi) == 4 ? bn : ((bn / 2 + unit - 1) / unit) * unit;
  begin = which == 0 ? 0 : mid;
  end = which == 0 ? mid : bn;
}

template <typename OT>
__device__ __forceinline__ void epilogue_store16(OT* p, const float (&v)[16], bool vec);
template <>
__device__ __forceinline__ void epilogue_store16<float>(float* p, const float (&v)[16], bool vec) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) p[i] = v[i];
  }
}
template <>
__device__ __forceinline__ void epilogue_store16<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[16], bool vec) {
  if (vec) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 u;
      __nv_bfloat162 a = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]), b = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
      __nv_bfloat162 c = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]), d = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
      u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
      u.z = *reinterpret_cast<uint32_t*>(&c); u.w = *reinterpret_cast<uint32_t*>(&d);
      reinterpret_cast<uint4*>(p)[i] = u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) p[i] = __float2bfloat16_rn(v[i]);
  }
}

// For the accumulating epilogue of a whole tile: the residual of the warp's first block of 32
// columns (lane: column, entries: the warp's 32 rows), asked for while the tile's products still run.
template <int BN, int EPI, typename OT>
__device__ __forceinline__ void epilogue_prefetch(float (&first)[32], int row, int n0, const OT* __restrict__ out, int ldo,
                                                  int rows_m, int rows_n, int c_begin) {
  if ((EPI != EPI_ACCUMULATE && EPI != EPI_ACCUMULATE_NORM) || n0 + BN > rows_n) return;
  const int lane = threadIdx.x & 31;
  const int row0 = row - lane;
  const int rows_valid = min(32, rows_m - row0);
  const OT* gbase = out + (size_t)row0 * ldo + n0 + lane + c_begin;
#pragma unroll
  for (int rr = 0; rr < 32; ++rr) first[rr] = rr < rows_valid ? gb::to_float<OT>(gbase[(size_t)rr * ldo]) : 0.f;
}

// A norm folded in in front of the product (EpilogueArgs::sums_in): 1/rms of the thread's token from the
// partial sums, in their order; 1 without such a norm. Asked for while the tile's products still run.
__device__ __forceinline__ float epilogue_row_scale(const EpilogueArgs& ra, int row, int rows_m) {
  if (ra.sums_in == nullptr || row >= rows_m) return 1.f;
  float t = 0.f;
  for (int i = 0; i < ra.tiles_in; ++i) t += ra.sums_in[(size_t)i * ra.sums_ld + row];
  return rsqrtf(t * ra.inv_width + ra.eps);
}

// The epilogue of one 128 x BN tile for the thread that owns token `row` (a TMEM lane): taddr is the
// lane's address of the tile's first column, n0 the tile's first output column (packed row for
// the SiLU-gate), turn this warp's 32 x 33 floats of shared memory. Two warps share a lane
// quarter: each takes the columns [c_begin, c_end) (multiples of 128); the rotation's epilogue, which
// needs whole heads, and the paths for ragged tiles are run by the first of them alone.
template <int BN, int EPI, typename OT>
__device__ __forceinline__ void epilogue_tile(uint32_t taddr, int row, int n0, OT* __restrict__ out, int ldo,
                                              int rows_m, int rows_n, bool vec, const EpilogueArgs& ra, float* turn,
                                              int c_begin, int c_end, const float (&first)[32], const float inv) {
  // EMIT: the norm behind this accumulating product is folded in. Every warp writes the sum of squares
  // of its columns of every token into a row of its own of sums_out (two rows per tile of BN columns).
  constexpr bool EMIT = EPI == EPI_ACCUMULATE_NORM;
  const int sums_row = 2 * (n0 / BN) + (c_begin != 0 ? 1 : 0);
  // Whole tiles, the usual case: 32 columns at a time, turned round in shared memory. A thread holds
  // a row of the accumulator, so stores straight from its registers touch 32 different lines per
  // instruction; after the turn a warp's instruction covers 32 consecutive columns of one row, and
  // the residual of all 32 rows is asked for before any of it is used.
  if ((EPI == EPI_STORE || EPI == EPI_ACCUMULATE || EMIT) && n0 + BN <= rows_n) {
    const int lane = threadIdx.x & 31;
    const int row0 = row - lane;                               // the warp's first row
    const int rows_valid = min(32, rows_m - row0);             // may be <= 0
    OT* gbase = out + (size_t)row0 * ldo + n0 + lane;
    constexpr bool ACC = EPI == EPI_ACCUMULATE || EMIT;
    float ssq = 0.f;                                           // EMIT: of the token row0 + lane
    __nv_bfloat16* hbase = EMIT ? ra.h_out + (size_t)row0 * ldo + n0 + lane : nullptr;
    // the residual of a block is asked for one block ahead; the first block's before the tile's
    // products have finished (first: the caller's prefetch)
    float old_cur[ACC ? 32 : 1];
    auto fetch = [&](float (&dst)[ACC ? 32 : 1], int c) {
      if (ACC) {
#pragma unroll
        for (int rr = 0; rr < 32; ++rr)
          dst[ACC ? rr : 0] = rr < rows_valid ? gb::to_float<OT>(gbase[(size_t)rr * ldo + c]) : 0.f;
      }
    };
    if (ACC) {
#pragma unroll
      for (int rr = 0; rr < 32; ++rr) old_cur[ACC ? rr : 0] = first[ACC ? rr : 0];
    }
    constexpr int BLOCKS = BN / 32 / (epilogue_warps(EPI) / 4);     // blocks of 32 columns per warp
    constexpr int UNROLL = ACC ? 1 : BLOCKS;                       // the folded norm's work needs the registers
#pragma unroll UNROLL
    for (int k = 0; k < BLOCKS; ++k) {
      const int c = c_begin + 32 * k;
      if (c >= c_end) break;
      uint32_t r[32];
      tmem_ld_32(taddr + c, r);
      if (ACC && k > 0) fetch(old_cur, c);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) turn[lane * 33 + j] = __uint_as_float(r[j]);
      __syncwarp();
      const float wv = EMIT ? ra.weight[n0 + c + lane] : 0.f;
#pragma unroll
      for (int rr = 0; rr < 32; ++rr) {
        float v = turn[rr * 33 + lane];
        if (ACC) v += old_cur[ACC ? rr : 0];
        if (rr < rows_valid) store_value<OT>(gbase + (size_t)rr * ldo + c, v);
        if (EMIT) {
          // the squares go back the way the values came: each lane then adds up its own token's
          if (rr < rows_valid) hbase[(size_t)rr * ldo + c] = __float2bfloat16_rn(v * wv);
          turn[rr * 33 + lane] = rr < rows_valid ? v * v : 0.f;
        }
      }
      if (EMIT) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j) ssq += turn[lane * 33 + j];
      }
      __syncwarp();
    }
    if (EMIT && row < rows_m) ra.sums_out[(size_t)sums_row * ra.sums_ld + row] = ssq;
    return;
  }
  if (EPI == EPI_SWIGLU && vec && (n0 >> 1) + BN / 2 <= rows_n) {
    // columns [128 q, 128 q + 64) of the tile are gate values, the next 64 the up values of the same
    // 64 features; 32 features at a time, 16-byte stores from the thread's own row
    const bool row_ok = row < rows_m;
    OT* prow = out + (size_t)(row_ok ? row : 0) * ldo + (n0 >> 1);
#pragma unroll 1
    for (int q = c_begin / 128; q < c_end / 128; ++q) {
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        uint32_t g_[32], u_[32];
        tmem_ld_32(taddr + q * 128 + c, g_);
        tmem_ld_32(taddr + q * 128 + 64 + c, u_);
        tmem_ld_wait();
        if (!row_ok) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            v[j] = silu_gate_fast(__uint_as_float(g_[h * 16 + j]) * inv, __uint_as_float(u_[h * 16 + j]) * inv);
          epilogue_store16<OT>(prow + q * 64 + c + h * 16, v, true);
        }
      }
    }
    return;
  }
  if (c_begin != 0) {              // what follows runs once per lane quarter
    if (EMIT && row < rows_m) ra.sums_out[(size_t)sums_row * ra.sums_ld + row] = 0.f;
    return;
  }
  if (EPI == EPI_ROPE) {
    // This thread holds one token's row: whole heads, so both channels of every rotation pair.
    const int hd = ra.head_dim, half = hd >> 1;
    const bool token_ok = row < rows_m;
    const int pos = token_ok ? ra.positions[row] : 0;
    const int req = token_ok ? ra.token_req[row] : 0;
    const float2* tab = ra.cs + (size_t)(token_ok ? row : 0) * half;      // this token's cosines and sines
#pragma unroll 1
    for (int hc = 0; hc < BN && n0 + hc < rows_n; hc += hd) {
      const int head = (n0 + hc) / hd;
      const bool rotate = ra.cs != nullptr && head < ra.heads + ra.kv_heads;
      __nv_bfloat16* dst = token_ok ? rope_destination(ra, row, req, pos, head, 0) : nullptr;
      const bool split_halves = rotate && !ra.interleaved && half >= 16;
#pragma unroll 1
      for (int dd = 0; dd < (split_halves ? half : hd); dd += 16) {
        uint32_t ra_[16], rb_[16];
        tmem_ld_16(taddr + hc + dd, ra_);
        if (split_halves) tmem_ld_16(taddr + hc + half + dd, rb_);
        tmem_ld_wait();
        if (!dst) continue;
        float a[16], b[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          a[j] = __uint_as_float(ra_[j]) * inv;
          b[j] = split_halves ? __uint_as_float(rb_[j]) * inv : 0.f;
        }
        if (split_halves) {
          // channels dd .. dd + 15 pair with half + dd ..
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 v = tab[dd + j];
            const float cs = v.x, sn = v.y;
            const float x = a[j], y = b[j];
            a[j] = x * cs - y * sn;
            b[j] = x * sn + y * cs;
          }
          epilogue_store16<__nv_bfloat16>(dst + dd, a, true);
          epilogue_store16<__nv_bfloat16>(dst + half + dd, b, true);
        } else {
          if (rotate) {
            // pairs inside the chunk: (2k, 2k + 1), or for a head of 16 channels (k, k + 8)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int ia = ra.interleaved ? 2 * k : k, ib = ra.interleaved ? 2 * k + 1 : k + 8;
              const float2 v = tab[ra.interleaved ? (dd >> 1) + k : k];
              const float cs = v.x, sn = v.y;
              const float x = a[ia], y = a[ib];
              a[ia] = x * cs - y * sn;
              a[ib] = x * sn + y * cs;
            }
          }
          epilogue_store16<__nv_bfloat16>(dst + dd, a, true);
        }
      }
    }
  } else if (EPI == EPI_SWIGLU) {
    // columns [128 q, 128 q + 64) of the tile are gate values, the next 64 the up values of
    // the same features: feature = 64 * (packed row / 128) + offset
#pragma unroll 1
    for (int q = 0; q < BN / 128; ++q) {
#pragma unroll 1
      for (int c = 0; c < 64; c += 16) {
        uint32_t r0[16], r1[16];
        tmem_ld_16(taddr + q * 128 + c, r0);
        tmem_ld_16(taddr + q * 128 + 64 + c, r1);
        tmem_ld_wait();
        const int col = (n0 >> 1) + q * 64 + c;      // output feature of the first of 16
        if (row >= rows_m || col >= rows_n) continue;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = silu_gate_fast(__uint_as_float(r0[j]) * inv, __uint_as_float(r1[j]) * inv);
        OT* p = out + (size_t)row * ldo + col;
        if (col + 16 <= rows_n) {
          epilogue_store16<OT>(p, v, vec);
        } else {
          for (int j = 0; j < 16 && col + j < rows_n; ++j) store_value<OT>(p + j, v[j]);
        }
      }
    }
  } else {
  float ssq = 0.f;
#pragma unroll 1
  for (int c = 0; c < BN; c += 16) {
    uint32_t r0[16];
    tmem_ld_16(taddr + c, r0);
    tmem_ld_wait();
    const int col = n0 + c;
    if (row >= rows_m || col >= rows_n) continue;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r0[j]) * inv;
    OT* p = out + (size_t)row * ldo + col;
    if (EMIT) {
      for (int j = 0; j < 16 && col + j < rows_n; ++j) {
        const float x = v[j] + gb::to_float<OT>(p[j]);
        store_value<OT>(p + j, x);
        ra.h_out[(size_t)row * ldo + col + j] = __float2bfloat16_rn(x * ra.weight[col + j]);
        ssq += x * x;
      }
      continue;
    }
    if (col + 16 <= rows_n) {
      if (EPI == EPI_ACCUMULATE) {
        if (vec) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 old = reinterpret_cast<const float4*>(p)[i];
            v[4 * i] += old.x; v[4 * i + 1] += old.y; v[4 * i + 2] += old.z; v[4 * i + 3] += old.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += gb::to_float<OT>(p[j]);
        }
      }
      epilogue_store16<OT>(p, v, vec);
    } else {
      for (int j = 0; j < 16 && col + j < rows_n; ++j) {
        float x = v[j];
        if (EPI == EPI_ACCUMULATE) x += gb::to_float<OT>(p[j]);
        store_value<OT>(p + j, x);
      }
    }
  }
  if (EMIT && row < rows_m) ra.sums_out[(size_t)sums_row * ra.sums_ld + row] = ssq;
  }
}

// EPI_SWIGLU: the weight rows are packed gate/up groups; rows_n counts the output features and the
// tiles run over the packed rows (twice as many).
template <int BN, int EPI, typename OT>
__global__ void __launch_bounds__(p_threads(EPI), 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_n,
                          OT* __restrict__ out, int ldo, int rows_m, int rows_n, int K, int tiles_m,
                          int tiles_n, const EpilogueArgs ra) {
  constexpr bool DUAL = false;
  using G = Geometry<BN, false, false, false>;
  constexpr int STAGES = G::STAGES;
  constexpr int ACC_COLS = G::ACCUMULATORS * BN;        // columns of one accumulator stage
  constexpr int TMEM_COLS = 2 * ACC_COLS;               // two stages: 256 or 512
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "two accumulator stages must fill a power of two");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ float turn_buf[epilogue_warps(EPI)][32 * 33];       // per epilogue warp: a 32 x 32 block on its way round

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int total_tiles = tiles_m * tiles_n;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), epilogue_warps(EPI));      // one arrival per epilogue warp
    }
    abort_s = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&map_m);
    prefetch_tensormap(&map_n);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* aborted = &abort_s;
  gb::pdl_launch_dependents();
  gb::pdl_wait();     // the activations, and for an accumulating epilogue the output, come from earlier kernels

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer
      int it = 0, issued = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*aborted; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) & 1) ^ 1)) {
            gb_err::report(ERR_WAIT_EMPTY);
            *aborted = 1;
          }
          if (*aborted) break;
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t base = tiles + s * G::STAGE_BYTES;
          mbar_arrive_expect_tx(bar, G::STAGE_BYTES);
          tma_load_2d(base, &map_m, bar, kb * BK, m0);
          tma_load_2d(base + G::A_BYTES, &map_n, bar, kb * BK, n0);
          issued = it + 1;
        }
      }
      if (*aborted) {
        for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j) {
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&full_bar[j % STAGES]), (j / STAGES) & 1)) {
            if (globaltimer_ns() - t0 > 20000000ull) {
              gb_err::report(ERR_WAIT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
      int it = 0, t = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*aborted; tile += gridDim.x, ++t) {
        const int as = t & 1;
        if (!mbar_wait(smem_u32(&acc_empty[as]), ((t >> 1) & 1) ^ 1)) {   // the epilogue has drained this stage
          gb_err::report(ERR_WAIT_ACCUM);
          *aborted = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + as * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) {
            gb_err::report(ERR_WAIT_FULL);
            *aborted = 1;
          }
          if (*aborted) break;
          tc_fence_after_sync();
          const uint32_t base = tiles + s * G::STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t koff = k * UMMA_K * 2;
            const bool accumulate = kb > 0 || k > 0;
            const uint64_t da = smem_desc_sw128(base + koff);
            mma_bf16(acc, da, smem_desc_sw128(base + G::A_BYTES + koff), idesc, accumulate);
          }
          mma_commit(smem_u32(&empty_bar[s]));
        }
        mma_commit(smem_u32(&acc_full[as]));
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32 * (warp % 4)
    int c_begin, c_end;
    epilogue_columns(EPI, BN, (warp - 2) >> 2, c_begin, c_end);
    const bool vec = (((uintptr_t)out) & 15) == 0 && ((size_t)ldo * sizeof(OT)) % 16 == 0;
    int t = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++t) {
      const int as = t & 1;
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      float first[32];
      epilogue_prefetch<BN, EPI, OT>(first, m0 + quarter * 32 + lane, n0, out, ldo, rows_m, rows_n, c_begin);
      const float inv = epilogue_row_scale(ra, m0 + quarter * 32 + lane, rows_m);
      bool have = mbar_wait(smem_u32(&acc_full[as]), (t >> 1) & 1);
      if (!have && lane == 0) {
        gb_err::report(ERR_WAIT_ACCUM);
        *aborted = 1;
      }
      if (!have || *aborted) break;
      tc_fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + as * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      epilogue_tile<BN, EPI, OT>(taddr, row, n0, out, ldo, rows_m, rows_n, vec, ra, turn_buf[warp - 2], c_begin, c_end, first, inv);
      // every read of this accumulator stage has completed: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// --------------------------------------------------------------------------
// Many tokens, CTA pairs: two CTAs of a cluster share 256 x 256 tiles. Each CTA loads its 128 token
// rows and its half (128 rows) of the weight tile; one thread of the even CTA issues products with
// M = 256 that read both CTAs' shared memory and leave each CTA's 128 rows in its own tensor memory.
// A CTA thus fetches 32 KB per 64-deep step instead of 48 KB for the same work: the stream of
// operands from L2 is cut by a third. Six (eight) stages; the two
// accumulator stages and the epilogue are as in the single-CTA kernel, each CTA for its own rows.
// Barriers: `full` lives in the even CTA and counts both CTAs' TMA bytes; `empty` and `acc_full`
// are completed in both CTAs at once by the issuer's commits; `acc_empty` lives in the even CTA and
// takes one arrival per epilogue warp of both CTAs.
// BN: the pair's tile width. 256 is what is launched: with 128 the products themselves took nearly
// twice as long per flop when measured (a pair's product of 128 columns costs about as much as one of
// 256), which outweighs hiding a lone tile's epilogue under a second tile; for the same reason tiles
// of 384 columns (a 256- and a 128-column product per step), tried for widths where 256-wide tiles
// need a second, nearly empty round over the pairs, were slower than that second round.
// BN = 320 (five heads of 64, for a query/key/value product whose 256-wide tiles would need a second,
// nearly empty round): a product has at most 256 columns, so a step is a product of 256 and one of
// 64 columns (two of 160 took longer: a product's time grows in steps with its width); each CTA
// loads its half of either product's weight rows, so that the accumulator's columns stay in the
// weights' order. 320 columns leave tensor memory for one accumulator stage only.
template <int BN>
struct PairGeometry {
  static constexpr int PARTS = BN > 256 ? 2 : 1;                           // products per step
  static constexpr int COLS0 = BN > 256 ? 256 : BN, COLS1 = BN - COLS0;    // their widths
  static constexpr int BOX_ROWS = BN > 256 ? COLS1 / 2 : BN / 2;           // weight rows per TMA box
  static constexpr int ACC_STAGES = 2 * BN <= 512 ? 2 : 1;
  static constexpr int STAGE_BYTES = BM * BK * 2 + (BN / 2) * BK * 2;      // per CTA: 32 KB, 24 KB or 36 KB
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;                // 6, 8 or 5
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static_assert(STAGE_BYTES % 1024 == 0 && (BOX_ROWS * BK * 2) % 1024 == 0 && (COLS0 / 2) % BOX_ROWS == 0,
                "operand tiles on swizzle boundaries, whole boxes");
};

template <int BN, int EPI, typename OT>
__global__ void __launch_bounds__(p_threads(EPI), 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_n,
                    OT* __restrict__ out, int ldo, int rows_m, int rows_n, int K, int tiles_m, int tiles_n,
                    const EpilogueArgs ra) {
  using PG = PairGeometry<BN>;
  constexpr int STAGES = PG::STAGES, PAIR_STAGE_BYTES = PG::STAGE_BYTES;
  constexpr int ACC = PG::ACC_STAGES;             // accumulator stages
  constexpr int TMEM_COLS = ACC * BN <= 512 && ACC * BN > 256 ? 512 : ACC * BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ float turn_buf[epilogue_warps(EPI)][32 * 33];       // per epilogue warp: a 32 x 32 block on its way round

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();         // 0: issues the products
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int num_kb = (K + BK - 1) / BK;
  const int total_tiles = tiles_m * tiles_n;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), 2 * epilogue_warps(EPI));      // one arrival per epilogue warp of both CTAs
    }
    abort_s = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&map_m);
    prefetch_tensormap(&map_n);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&tmem_base_s), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive_wait();        // both CTAs' barriers exist before either signals the other's
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* aborted = &abort_s;
  gb::pdl_launch_dependents();
  gb::pdl_wait();     // the activations, and for an accumulating epilogue the output, come from earlier kernels

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ producer (both CTAs)
      int s = 0, par = 1, issued = 0;
      for (int tile = pair; tile < total_tiles && !*aborted; tile += pairs) {
        const int m0 = (tile % tiles_m) * (2 * BM) + (int)rank * BM;
        const int nt0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[s]), par)) {
            gb_err::report(ERR_WAIT_EMPTY);
            *aborted = 1;
          }
          if (*aborted) break;
          const uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);     // the even CTA's barrier
          const uint32_t base = tiles + s * PAIR_STAGE_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * PAIR_STAGE_BYTES);
          tma_load_2d_pair(base, &map_m, bar, kb * BK, m0);
          // this CTA's half of the first product's weight rows, then of the second's, box by box
#pragma unroll
          for (int b = 0; b < BN / 2 / PG::BOX_ROWS; ++b) {
            const int r0 = b * PG::BOX_ROWS;      // row within this CTA's BN / 2
            const int feature = r0 < PG::COLS0 / 2 ? (int)rank * (PG::COLS0 / 2) + r0
                                                   : PG::COLS0 + (int)rank * (PG::COLS1 / 2) + (r0 - PG::COLS0 / 2);
            tma_load_2d_pair(base + BM * BK * 2 + r0 * BK * 2, &map_n, bar, kb * BK, nt0 + feature);
          }
          ++issued;
          if (++s == STAGES) s = 0, par ^= 1;
        }
      }
      if (*aborted && issued > 0) {
        // wind down: the copies in flight (counted on the even CTA's barriers) need microseconds
        // to land; give them two milliseconds before the CTA's shared memory is given up
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------------------------------------ MMA issuer (even CTA)
      constexpr uint32_t idesc = instr_desc_bf16(2 * BM, PG::COLS0);
      constexpr uint32_t idesc1 = instr_desc_bf16(2 * BM, PG::COLS1 > 0 ? PG::COLS1 : 16);
      const uint64_t da0 = smem_desc_sw128(tiles), db0 = smem_desc_sw128(tiles + BM * BK * 2);
      int s = 0, par = 0, t = 0;
      for (int tile = pair; tile < total_tiles && !*aborted; tile += pairs, ++t) {
        const int as = ACC == 2 ? (t & 1) : 0;
        if (!mbar_wait(smem_u32(&acc_empty[as]), ((ACC == 2 ? (t >> 1) : t) & 1) ^ 1)) {   // both epilogues have drained this stage
          gb_err::report(ERR_WAIT_ACCUM);
          *aborted = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + as * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[s]), par)) {
            gb_err::report(ERR_WAIT_FULL);
            *aborted = 1;
          }
          if (*aborted) break;
          tc_fence_after_sync();
          const uint64_t da = da0 + (uint64_t)(s * (PAIR_STAGE_BYTES >> 4)), db = db0 + (uint64_t)(s * (PAIR_STAGE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            mma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, kb > 0 || k > 0);
            if (PG::PARTS == 2)
              mma_bf16_pair(acc + PG::COLS0, da + 2 * k, db + (uint64_t)((PG::COLS0 / 2) * BK * 2 >> 4) + 2 * k, idesc1,
                            kb > 0 || k > 0);
          }
          mma_commit_pair(smem_u32(&empty_bar[s]), 3);      // the stage is free in both CTAs
          if (++s == STAGES) s = 0, par ^= 1;
        }
        mma_commit_pair(smem_u32(&acc_full[as]), 3);
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue warps (both CTAs, own rows)
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32 * (warp % 4)
    int c_begin, c_end;
    epilogue_columns(EPI, BN, (warp - 2) >> 2, c_begin, c_end);
    const bool vec = (((uintptr_t)out) & 15) == 0 && ((size_t)ldo * sizeof(OT)) % 16 == 0;
    int t = 0;
    for (int tile = pair; tile < total_tiles; tile += pairs, ++t) {
      const int as = ACC == 2 ? (t & 1) : 0;
      const int m0 = (tile % tiles_m) * (2 * BM) + (int)rank * BM, n0 = (tile / tiles_m) * BN;
      float first[32];
      epilogue_prefetch<BN, EPI, OT>(first, m0 + quarter * 32 + lane, n0, out, ldo, rows_m, rows_n, c_begin);
      const float inv = epilogue_row_scale(ra, m0 + quarter * 32 + lane, rows_m);
      bool have = mbar_wait(smem_u32(&acc_full[as]), (ACC == 2 ? (t >> 1) : t) & 1);
      if (!have && lane == 0) {
        gb_err::report(ERR_WAIT_ACCUM);
        *aborted = 1;
      }
      if (!have || *aborted) break;
      tc_fence_after_sync();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + as * BN + ((uint32_t)(quarter * 32) << 16);
      epilogue_tile<BN, EPI, OT>(taddr, row, n0, out, ldo, rows_m, rows_n, vec, ra, turn_buf[warp - 2], c_begin, c_end, first, inv);
      // every read of this accumulator stage has completed: hand it back to the issuer
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(smem_u32(&acc_empty[as]));
        else mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[as]), 0));
      }
    }
  }
  // Neither CTA may leave, or give its tensor memory back, while the other's products or copies may
  // still touch it.
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive_wait();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side
// How many CTAs of a cluster share K. Measured on B200 (2048- to 5632-wide layers, 8 tokens): a CTA
// costs about 3.5 us before and after its stream of K blocks and streams one 16 KB block in about
// 0.26 us, so the fixed part weighs as much as 13 blocks; two CTAs on one SM halve each other's rate,
// so the CTAs should not outnumber the SMs; clusters of more than six are placed badly.
// `active[s]`: whether clusters of size s can be resident at all (0: not asked yet, -1: no), kept by the
// caller per kernel.
struct ClusterPlan { int split, stages; };

// The cost of a plan in units of one K block's streaming time: a CTA costs about 13.5 blocks of set-up,
// first-byte latency, reduction and tail besides its own blocks (timeline measurements). Two ways to
// place the CTAs: one per SM with the full pipeline, or, with a pipeline short enough for two CTAs
// to share an SM's shared memory, up to two per SM; CTAs that share an SM also share its path to L2:
// 1.3 to 1.65 times the time of a CTA that has the SM to itself, by how many SMs hold two.
template <typename Kernel, typename G>
ClusterPlan pick_cluster_plan(Kernel kernel, int* active, int tiles, int total_kb) {
  ClusterPlan best{1, G::STAGES};
  double best_cost = 1e30;
  const int sms = sm_count();
  for (int s = 1; s <= G::MAX_CLUSTER && s <= 6 && s <= total_kb; ++s) {
    const int st1 = G::stages_that_fit(s);       // one CTA per SM: as deep a pipeline as fits
    if (st1 < 2) continue;
    if (active[s] == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1, 148, s);
      cfg.blockDim = dim3(C_THREADS);
      cfg.dynamicSmemBytes = G::smem_bytes(s, st1);
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = s;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = -1;
      }
      active[s] = n;
    }
    if (active[s] < 1) continue;
    const int per = (total_kb + s - 1) / s;
    const int ctas = tiles * s;
    // one CTA per SM; whole clusters must find room in one GPC, so fewer may be resident than
    // the SMs would hold CTAs
    {
      const int rounds = (tiles + active[s] - 1) / active[s];
      const double cost = (double)rounds * (per + 13.5);
      if (cost < best_cost) { best_cost = cost; best = ClusterPlan{s, st1}; }
    }
    // two per SM: the most stages that let two CTAs (and their 1 KB each of reserve) share 227 KB
    int st2 = G::STAGES;
    while (st2 > 2 && 2 * (G::smem_bytes(s, st2) + 2048) > SMEM_LIMIT) --st2;
    if (2 * (G::smem_bytes(s, st2) + 2048) <= SMEM_LIMIT && ctas > sms) {
      const double share = 2 * ctas <= 3 * sms ? 1.3 : 1.65;      // measured at 1.2 and 1.8 CTAs per SM
      const double cost = (double)((ctas + 2 * sms - 1) / (2 * sms)) * (per + 13.5) * share;
      if (cost < best_cost) { best_cost = cost; best = ClusterPlan{s, st2}; }
    }
  }
  return best;
}

// weight_rows: rows of the weight matrix as stored (for the SiLU-gate epilogue the packed rows,
// twice the output features); out_features: columns of the output.
template <int BN, int EPI, typename OT>
int launch_cluster(const CUtensorMap& mm, const CUtensorMap& mn, OT* out, int ldo, int weight_rows, int out_features,
                   int tokens, int K, cudaStream_t stream, const EpilogueArgs& ra = EpilogueArgs{}) {
  using G = Geometry<BN, false, false, true, rope_table_bytes(EPI, BN)>;
  auto kernel = gemm_tc_cluster_kernel<BN, EPI, OT>;
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         G::most_smem());
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(e));
    configured.done();
  }
  const int tiles_n = (tokens + BN - 1) / BN, tiles_m = (weight_rows + BM - 1) / BM;
  const int total_kb = (K + BK - 1) / BK;
  static int active[9] = {0};
  const ClusterPlan plan = pick_cluster_plan<decltype(kernel), G>(kernel, active, tiles_n * tiles_m, total_kb);
  int split = plan.split;
  const int per = (total_kb + split - 1) / split;
  split = (total_kb + per - 1) / per;            // no rank without K blocks
  return gb::check_pdl_launch(gb::launch_pdl(kernel, dim3(tiles_n, tiles_m, split), dim3(C_THREADS),
                                             G::smem_bytes(split, plan.stages), stream, dim3(1, 1, split), mm, mn, out, ldo,
                                             out_features, tokens, K, per, ra, plan.stages),
                              "gemm_tc (cluster)");
}

// Few tokens: the weights are the MMA-row operand; BN tokens per tile.
template <int BN>
int dispatch_cluster(int epi, int out_dtype, const CUtensorMap& mm, const CUtensorMap& mn, void* out, int ldo,
                     int weight_rows, int out_features, int tokens, int K, cudaStream_t stream, const EpilogueArgs& ra) {
  if (epi == EPI_STORE) {
    if (out_dtype == GB_F32)
      return launch_cluster<BN, EPI_STORE, float>(mm, mn, (float*)out, ldo, weight_rows, out_features, tokens, K, stream, ra);
    return launch_cluster<BN, EPI_STORE, __nv_bfloat16>(mm, mn, (__nv_bfloat16*)out, ldo, weight_rows, out_features, tokens, K, stream, ra);
  }
  if (epi == EPI_ACCUMULATE && ra.h_out != nullptr)
    return launch_cluster<BN, EPI_ACCUMULATE_NORM, float>(mm, mn, (float*)out, ldo, weight_rows, out_features, tokens, K, stream, ra);
  if (epi == EPI_ACCUMULATE)
    return launch_cluster<BN, EPI_ACCUMULATE, float>(mm, mn, (float*)out, ldo, weight_rows, out_features, tokens, K, stream, ra);
  return launch_cluster<BN, EPI_SWIGLU, __nv_bfloat16>(mm, mn, (__nv_bfloat16*)out, ldo, weight_rows, out_features, tokens, K, stream, ra);
}

template <int BN, int EPI, typename OT>
int launch_persistent(const CUtensorMap& mm, const CUtensorMap& mn, OT* out, int ldo, int tokens, int weight_rows,
                      int out_features, int K, cudaStream_t stream, const EpilogueArgs& ra = EpilogueArgs{}) {
  using G = Geometry<BN, false, false, false>;
  auto kernel = gemm_tc_persistent_kernel<BN, EPI, OT>;
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(e));
    configured.done();
  }
  const int tiles_m = (tokens + BM - 1) / BM, tiles_n = (weight_rows + BN - 1) / BN;
  const int total = tiles_m * tiles_n;
  const int grid = total < sm_count() ? total : sm_count();
  return gb::check_pdl_launch(gb::launch_pdl(kernel, dim3(grid), dim3(p_threads(EPI)), G::SMEM_BYTES, stream, dim3(1, 1, 1), mm, mn, out,
                                             ldo, tokens, out_features, K, tiles_m, tiles_n, ra),
                              "gemm_tc (persistent)");
}

// 256 x BN tiles on CTA pairs (clusters of two).
template <int BN, int EPI, typename OT>
int launch_pair(const CUtensorMap& mm, const CUtensorMap& mn, OT* out, int ldo, int tokens, int weight_rows,
                int out_features, int K, cudaStream_t stream, const EpilogueArgs& ra = EpilogueArgs{}) {
  using PG = PairGeometry<BN>;
  auto kernel = gemm_tc_pair_kernel<BN, EPI, OT>;
  static gb::OncePerDevice configured;
  if (configured.needed()) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PG::SMEM_BYTES);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(e));
    configured.done();
  }
  const int tiles_m = (tokens + 2 * BM - 1) / (2 * BM), tiles_n = (weight_rows + BN - 1) / BN;
  const int total = tiles_m * tiles_n, most = sm_count() / 2;
  const int pairs = total < most ? total : most;
  return gb::check_pdl_launch(gb::launch_pdl(kernel, dim3(2 * pairs), dim3(p_threads(EPI)), PG::SMEM_BYTES, stream, dim3(2, 1, 1),
                                             mm, mn, out, ldo, tokens, out_features, K, tiles_m, tiles_n, ra),
                              "gemm_tc (pairs)");
}

// Tile width for many tokens: the one that needs fewer rounds over the SMs (a 256-wide tile costs
// two 128-wide ones but reads each operand half as often); ties go to the wide tile.
int pick_tile_width(int rows_m, int rows_n) {
  const int tiles_m = (rows_m + BM - 1) / BM, sms = sm_count();
  auto cost = [&](int bn) {
    const int tiles = tiles_m * ((rows_n + bn - 1) / bn);
    return (long long)((tiles + sms - 1) / sms) * bn;
  };
  return cost(256) <= cost(128) ? 256 : 128;
}

// Up to this many tokens the weights are the MMA's rows and clusters split K (see the head of this file);
// more tokens than one tile's 64 columns make several column tiles, each of which reads the weights
// (from L2 after the first). With the TinyLlama layer sizes a step of 65 to 256 tokens took 2.1 to 2.8 ms
// this way against 2.9 to 3.5 ms with 128-row token tiles, which are too few CTAs to stream the weights;
// from about 400 tokens on the two are level.
constexpr int few_token_limit() { return 256; }

// More than 64 tokens: whether CTA pairs take the product, and the tile width over the weight's rows.
// Pairs pay from about a thousand tokens (768: 3.9 ms a step with pairs, 3.4 without; 1,024: 4.4 against 4.5):
// below that their 256 x 256 tiles are too few for the 74 pairs.
bool many_token_pairs(int tokens, int weight_rows, int epi = -1) {
  if (weight_rows < 256) return false;
  if (tokens >= 8 * BM) return true;
  // The gate/up product has the most tiles by far, and below a thousand tokens still pays where the
  // pairs' 256 x 256 tiles need fewer rounds: a round of pairs costs a CTA as much as a round of 128-wide
  // tiles (1 MB of operands for each), so 512 tokens times 11,264 packed rows are two rounds of pairs
  // against three (a step of 512 tokens 3.35 to 3.1 ms). The other products have one round either way.
  if (epi != EPI_SWIGLU || tokens <= few_token_limit()) return false;
  const int sms = sm_count(), pairs = sms / 2;
  const int pair_tiles = ((tokens + 2 * BM - 1) / (2 * BM)) * ((weight_rows + 255) / 256);
  const int pair_cost = ((pair_tiles + pairs - 1) / pairs) * 128;
  const int tiles_m = (tokens + BM - 1) / BM;
  auto cost = [&](int bn) { return ((tiles_m * ((weight_rows + bn - 1) / bn) + sms - 1) / sms) * bn; };
  return pair_cost < (cost(256) < cost(128) ? cost(256) : cost(128));
}
int many_token_width(int tokens, int weight_rows, int epi = -1) {
  return many_token_pairs(tokens, weight_rows, epi) ? 256 : pick_tile_width(tokens, weight_rows);
}

}  // namespace

GB_DEFINE_LAST_ERROR()

// Returns the device error word (0: none) and clears it. Synchronises the device.
GB_EXPORT int gb_tc_error_check() { return gb_err::fetch_and_clear(); }

// A word of pinned host memory that a kernel's failed wait also writes its code to (null: none).
GB_EXPORT int gb_tc_set_error_sink(int* host_word) { return gb_err::set_sink(host_word); }

namespace {
// One warp waits, for at most limit_ns, on a barrier that nothing will ever complete.
__global__ void wait_that_runs_out_kernel(unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait(smem_u32(&bar), 0, limit_ns)) gb_err::report(ERR_WAIT_FULL);
}
}  // namespace

// For tests of the error path: launches a kernel whose one wait runs out after limit_us
// microseconds (at most 100 ms), which then records its code as any product kernel would and returns.
GB_EXPORT int gb_tc_selftest_wait_runs_out(int limit_us, cudaStream_t stream) {
  if (limit_us < 1 || limit_us > 100000) return gb::fail(GB_BAD_ARGUMENT, "the limit must be 1 to 100000 us");
  wait_that_runs_out_kernel<<<1, 32, 0, stream>>>((unsigned long long)limit_us * 1000ull);
  return gb::check_launch("wait_that_runs_out");
}

// An RMS norm folded into the products around it (see EpilogueArgs). As the consumer: sums_in
// [tiles_in, sums_ld] and eps, inv_width = 1 / features of the normed vector. As the producer
// (accumulating products only): h_out [Mx, Nw] bfloat16, weight [Nw] 32-bit, sums_out
// [gb_gemm_tc_norm_tiles(Mx, Nw), sums_ld]. Unused halves are null.
struct GbNormFold {
  const float* sums_in;
  int tiles_in;
  float eps, inv_width;
  void* h_out;
  const float* weight;
  float* sums_out;
  int sums_ld;
};

namespace {
thread_local const void* g_next_stream = nullptr;
thread_local long long g_next_bytes = 0;
// the hint is for one launch: taken and cleared
void take_next_stream(EpilogueArgs& ra) {
  ra.next_stream = (const uint8_t*)g_next_stream;
  ra.next_bytes = g_next_bytes;
  g_next_stream = nullptr;
  g_next_bytes = 0;
}
void fold_norm(EpilogueArgs& ra, const GbNormFold* n) {
  if (n == nullptr) return;
  ra.sums_in = n->sums_in; ra.tiles_in = n->tiles_in; ra.eps = n->eps; ra.inv_width = n->inv_width;
  ra.h_out = (__nv_bfloat16*)n->h_out; ra.weight = n->weight; ra.sums_out = n->sums_out; ra.sums_ld = n->sums_ld;
}
}  // namespace

// A hint for the calling thread's next product: the weights (16-byte aligned) that the kernel after
// it will stream, which its CTAs then ask to be brought into L2 while they wait out their own
// latencies. Only the few-token kernels act on it. Null or 0 bytes: no hint.
GB_EXPORT int gb_tc_hint_next_stream(const void* weights, long long bytes) {
  if (((uintptr_t)weights & 15) != 0) return gb::fail(GB_BAD_ARGUMENT, "the hinted weights are not 16-byte aligned");
  g_next_stream = bytes > 0 ? weights : nullptr;
  g_next_bytes = bytes > 0 ? bytes : 0;
  return GB_OK;
}

// Rows of sums_out that a product of Mx tokens and Nw output features writes when a norm is folded
// in behind it; 0: this shape does not fold norms.
GB_EXPORT int gb_gemm_tc_norm_tiles(int Mx, int Nw) {
  if (Mx <= few_token_limit()) return (Nw + BM - 1) / BM;                   // a row per tile of 128 features
  const int width = many_token_width(Mx, Nw);
  return 2 * ((Nw + width - 1) / width);                      // a row per epilogue warp of a lane quarter
}

// Whether gb_gemm_tc takes this problem (else the caller uses the plain kernel).
GB_EXPORT int gb_gemm_tc_supported(const void* x, const void* w, int Mx, int Nw, int K) {
  if (Mx < 1 || Nw < 1 || K < 8 || K % 8) return 0;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return 0;
  return 1;
}

// epi 0: out[Mx,Nw] = x w^T (out_dtype f32 or bf16); 1: out (f32) += x w^T;
// 2: w holds gate and up rows packed in groups of 64 ([128 * ceil(Nw / 64), K], see the head of this
// file); out[Mx,Nw] (bf16) = silu(x gate^T) * (x up^T).
GB_EXPORT int gb_gemm_tc(const void* x, const void* w, void* out, int Mx, int Nw, int K, int out_dtype, int epi,
                         const GbNormFold* norm, cudaStream_t stream) {
  if (!gb_gemm_tc_supported(x, w, Mx, Nw, K))
    return gb::fail(GB_UNSUPPORTED, "gemm_tc: needs K a multiple of 8 and 16-byte aligned operands (K = %d)", K);
  if (epi == EPI_ACCUMULATE && out_dtype != GB_F32)
    return gb::fail(GB_BAD_ARGUMENT, "gemm_tc: accumulation needs a 32-bit output");
  if (epi == EPI_SWIGLU && out_dtype != GB_BF16)
    return gb::fail(GB_BAD_ARGUMENT, "gemm_tc: the SiLU-gate epilogue writes bfloat16");
  const int weight_rows = epi == EPI_SWIGLU ? 128 * ((Nw + 63) / 64) : Nw;
  EpilogueArgs ra{};
  fold_norm(ra, norm);
  take_next_stream(ra);
  if (ra.h_out != nullptr && epi != EPI_ACCUMULATE)
    return gb::fail(GB_UNSUPPORTED, "gemm_tc: a norm is folded in behind accumulating products only (epilogue %d)", epi);
  CUtensorMap mm, mn;
  int rc;
  if (Mx <= few_token_limit()) {
    const int bn = Mx <= 16 ? 16 : Mx <= 32 ? 32 : 64;
    if ((rc = tensor_map_2d(w, weight_rows, K, BM, &mm))) return rc;
    if ((rc = tensor_map_2d(x, Mx, K, bn, &mn))) return rc;
    if (bn == 16) return dispatch_cluster<16>(epi, out_dtype, mm, mn, out, Nw, weight_rows, Nw, Mx, K, stream, ra);
    if (bn == 32) return dispatch_cluster<32>(epi, out_dtype, mm, mn, out, Nw, weight_rows, Nw, Mx, K, stream, ra);
    return dispatch_cluster<64>(epi, out_dtype, mm, mn, out, Nw, weight_rows, Nw, Mx, K, stream, ra);
  }
  if ((rc = tensor_map_2d(x, Mx, K, BM, &mm))) return rc;
  const bool pairs = many_token_pairs(Mx, weight_rows, epi);
  const int width = many_token_width(Mx, weight_rows, epi);
  // CTA pairs: each CTA of a pair loads half of the weight tile's rows
  if ((rc = tensor_map_2d(w, weight_rows, K, pairs ? 128 : width, &mn))) return rc;
#define GB_MANY(LAUNCH, BN_)                                                                                          \
  do {                                                                                                                \
    if (epi == EPI_SWIGLU)                                                                                            \
      return LAUNCH<BN_, EPI_SWIGLU, __nv_bfloat16>(mm, mn, (__nv_bfloat16*)out, Nw, Mx, weight_rows, Nw, K, stream, ra); \
    if (epi == EPI_ACCUMULATE && ra.h_out != nullptr)                                                                 \
      return LAUNCH<BN_, EPI_ACCUMULATE_NORM, float>(mm, mn, (float*)out, Nw, Mx, weight_rows, Nw, K, stream, ra);    \
    if (epi == EPI_ACCUMULATE)                                                                                        \
      return LAUNCH<BN_, EPI_ACCUMULATE, float>(mm, mn, (float*)out, Nw, Mx, weight_rows, Nw, K, stream, ra);         \
    if (out_dtype == GB_F32)                                                                                          \
      return LAUNCH<BN_, EPI_STORE, float>(mm, mn, (float*)out, Nw, Mx, weight_rows, Nw, K, stream, ra);              \
    return LAUNCH<BN_, EPI_STORE, __nv_bfloat16>(mm, mn, (__nv_bfloat16*)out, Nw, Mx, weight_rows, Nw, K, stream, ra); \
  } while (0)
  if (pairs) GB_MANY(launch_pair, 256);
  if (width == 256) GB_MANY(launch_persistent, 256);
  GB_MANY(launch_persistent, 128);
#undef GB_MANY
}

// The query/key/value product with the rotation and the cache write in its epilogue:
// x [Mx, K] times w [(heads + 2 kv_heads) * head_dim, K]^T; rotated queries to q_out [Mx, heads,
// head_dim], rotated keys and raw values into their pages (all bfloat16). cos_sin: [Mx, head_dim / 2, 2]
// cosines and sines of every token's angles (rope_table in elementwise.cu), or null: no rotation.
// head_dim must divide 128 (so that no head straddles a tile); returns GB_UNSUPPORTED otherwise.
GB_EXPORT int gb_gemm_tc_qkv(const void* x, const void* w, int Mx, int K, void* q_out, void* k_pool, void* v_pool,
                             const int32_t* positions, const int32_t* token_req, const int32_t* block_table,
                             int table_width, int heads, int kv_heads, int head_dim, const float* cos_sin,
                             int interleaved, int page_size, const GbNormFold* norm, cudaStream_t stream) {
  const int Nw = (heads + 2 * kv_heads) * head_dim;
  if (!gb_gemm_tc_supported(x, w, Mx, Nw, K))
    return gb::fail(GB_UNSUPPORTED, "gemm_tc: needs K a multiple of 8 and 16-byte aligned operands (K = %d)", K);
  if (head_dim < 16 || 128 % head_dim || head_dim % 16)
    return gb::fail(GB_UNSUPPORTED, "gemm_tc_qkv: head_dim %d does not divide 128", head_dim);
  if (kv_heads > 0 && (!k_pool || !v_pool || !block_table || page_size < 1))
    return gb::fail(GB_BAD_ARGUMENT, "gemm_tc_qkv: kv heads given without a cache to store them in");
  EpilogueArgs ra{};
  fold_norm(ra, norm);
  take_next_stream(ra);
  if (ra.h_out != nullptr)
    return gb::fail(GB_UNSUPPORTED, "gemm_tc_qkv: no norm can be folded in behind this product");
  ra.q_out = (__nv_bfloat16*)q_out; ra.k_pool = (__nv_bfloat16*)k_pool; ra.v_pool = (__nv_bfloat16*)v_pool;
  ra.positions = positions; ra.token_req = token_req; ra.block_table = block_table; ra.cs = reinterpret_cast<const float2*>(cos_sin);
  ra.table_width = table_width; ra.heads = heads; ra.kv_heads = kv_heads; ra.head_dim = head_dim;
  ra.interleaved = interleaved; ra.page_size = page_size;
  CUtensorMap mm, mn;
  int rc;
  __nv_bfloat16* none = nullptr;
  if (Mx <= few_token_limit()) {
    const int bn = Mx <= 16 ? 16 : Mx <= 32 ? 32 : 64;
    if ((rc = tensor_map_2d(w, Nw, K, BM, &mm))) return rc;
    if ((rc = tensor_map_2d(x, Mx, K, bn, &mn))) return rc;
    if (bn == 16) return launch_cluster<16, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Nw, Nw, Mx, K, stream, ra);
    if (bn == 32) return launch_cluster<32, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Nw, Nw, Mx, K, stream, ra);
    return launch_cluster<64, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Nw, Nw, Mx, K, stream, ra);
  }
  if ((rc = tensor_map_2d(x, Mx, K, BM, &mm))) return rc;
  if (many_token_pairs(Mx, Nw)) {
    // 320-wide tiles (two products a step, about 1.4 times a 256-wide tile's time) where they save a
    // round over the pairs: 2,048 tokens times 2,560 features are 80 tiles of 256 columns for 74 pairs,
    // but 64 of 320
    const int most = sm_count() / 2, tiles_m = (Mx + 2 * BM - 1) / (2 * BM);
    const int rounds256 = (tiles_m * ((Nw + 255) / 256) + most - 1) / most;
    const int rounds320 = (tiles_m * ((Nw + 319) / 320) + most - 1) / most;
    if (320 % head_dim == 0 && rounds320 * 14 < rounds256 * 10) {
      if ((rc = tensor_map_2d(w, Nw, K, PairGeometry<320>::BOX_ROWS, &mn))) return rc;
      return launch_pair<320, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Mx, Nw, Nw, K, stream, ra);
    }
    if ((rc = tensor_map_2d(w, Nw, K, 128, &mn))) return rc;
    return launch_pair<256, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Mx, Nw, Nw, K, stream, ra);
  }
  const int width = pick_tile_width(Mx, Nw);
  if ((rc = tensor_map_2d(w, Nw, K, width, &mn))) return rc;
  if (width == 256) return launch_persistent<256, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Mx, Nw, Nw, K, stream, ra);
  return launch_persistent<128, EPI_ROPE, __nv_bfloat16>(mm, mn, none, 0, Mx, Nw, Nw, K, stream, ra);
}
