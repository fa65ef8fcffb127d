// Causal grouped-query attention over the paged cache for prompt portions on the
// fifth-generation tensor cores: both matrix products of a tile are tcgen05.mma with
// accumulators in tensor memory, operands arrive by TMA, the softmax runs in 32-bit in
// registers between them.
//
// garuda/src/llama/mod.rs:793-818: s_j = dot(q, K_j) * scale over keys [start, pos],
// softmax with the maximum subtracted, sum of p_j V_j; query head h reads kv head h / g;
// start = max(0, pos + 1 - window) with a window (garuda/src/cache/mod.rs:333-338).
//
// One CTA takes 128 query rows, (token, head-of-group) pairs that share one kv head of
// one request, and walks the keys in tiles of 128:
//   warp 0   one lane: TMA. The query tile once (a 3-D box [tokens][group][64]); per key
//            tile one 4-D box per page for keys and for values, three stages.
//   warp 1   one lane: S = Q K^T into one of two S buffers in tensor memory (128 columns
//            each); after the softmax of a tile, O_tile = P V into one of two O buffers
//            (64 columns each). V is read as it lies in the cache, keys along the rows
//            (an MN-major operand).
//   warps 2-5  a thread owns a query row: reads its 128 scores from tensor memory, masks
//            (only on tiles that touch a row's limits), running maximum, exp2 with the
//            scale folded in, writes P in bfloat16 into shared memory in the layout the
//            second product reads (128-byte swizzle), and adds the previous tile's
//            O_tile, rescaled, to its 64 sums in registers.
// The S product of tile j + 1 runs while tile j is in the softmax; O_tile j is folded in
// after the softmax of tile j + 1, so the tensor cores never wait for the fold.
// Every wait is bounded; a wait that runs out sets the error word and the CTA winds down.
//
// Built for head size 64 only (one 128-byte swizzled row per key); other head sizes use the
// mma.sync kernels.
#include "attention_common.cuh"
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
constexpr int STAGES = 3;
constexpr int ROW_BYTES = HD * 2;   // 128: one swizzled row
constexpr int Q_BYTES = QROWS * ROW_BYTES;
constexpr int K_BYTES = KT * ROW_BYTES, V_BYTES = K_BYTES;
constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
constexpr int P_BYTES = QROWS * KT * 2;             // two blocks of 64 keys, [128 rows][128 bytes] each
constexpr int SMEM_BYTES = 1024 + Q_BYTES + STAGES * STAGE_BYTES + 2 * P_BYTES;
constexpr int TMEM_COLS = 512;                      // S: 2 x 128 columns, O: 2 x 64 columns
constexpr int O_COL0 = 256;
constexpr int THREADS = 192;

__device__ int g_tc_error_word;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tile_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, kv_full[STAGES], kv_empty[STAGES], s_ready[2], p_ready[2], o_ready[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.z, kvh = blockIdx.y;
  // The batch's lengths and block tables were copied in before the step's first kernel.
  const int q_begin = p.cu_q[r], q_len = p.cu_q[r + 1] - q_begin;
  if (q_len * p.g <= attn::ROWS_DECODE) return;      // a decode request: the other kernel's
  const int tokens_per_tile = QROWS / p.g;
  const int tok0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * tokens_per_tile;   // the longest tiles start first
  if (tok0 >= q_len) return;
  const int kv_len = p.kv_lens[r];
  const int32_t* table = p.block_table + (size_t)r * p.table_width;
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int nrows = ntok * p.g;
  const int pos0 = kv_len - q_len + tok0;                          // position of the tile's first token
  const int lo = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;   // first key any row reads
  const int hi = pos0 + ntok - 1;                                  // last key any row reads
  const int tile_begin = lo / KT, n_tiles = hi / KT + 1 - tile_begin;

  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = tiles;
  const uint32_t kv_s = tiles + Q_BYTES;                           // stage s: K at kv_s + s * STAGE_BYTES, V after it
  const uint32_t p_s = kv_s + STAGES * STAGE_BYTES;                // buffer b at p_s + b * P_BYTES

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_ready[b]), 1);
      mbar_init(smem_u32(&p_ready[b]), 128);
      mbar_init(smem_u32(&o_ready[b]), 1);
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
      mbar_arrive_expect_tx(smem_u32(&q_full), Q_BYTES);
      tma_load_3d(q_s, &q_map, smem_u32(&q_full), 0, kvh * p.g, q_begin + tok0);
      const int pages_per_tile = KT / p.page_size;
      const uint32_t page_bytes = (uint32_t)p.page_size * ROW_BYTES;
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % STAGES;
        if (j >= STAGES && !mbar_wait(smem_u32(&kv_empty[s]), ((j / STAGES) & 1) ^ 1)) {
          atomicCAS(&g_tc_error_word, 0, ERR_WAIT_EMPTY);
          abort_s = 1;
        }
        if (*(volatile int*)&abort_s) break;
        const int key0 = (tile_begin + j) * KT;
        const uint32_t bar = smem_u32(&kv_full[s]);
        const uint32_t kdst = kv_s + s * STAGE_BYTES, vdst = kdst + K_BYTES;
        // pages that hold a key some row reads, and exist
        int pages[16], count = 0;
        for (int g = 0; g < pages_per_tile; ++g) {
          const int first = key0 + g * p.page_size;
          pages[g] = (first <= hi && first + p.page_size > lo) ? table[first / p.page_size] : -1;
          count += pages[g] >= 0;
        }
        if (count == 0) {
          mbar_arrive(bar);
        } else {
          mbar_arrive_expect_tx(bar, 2u * count * page_bytes);
          for (int g = 0; g < pages_per_tile; ++g) {
            if (pages[g] < 0) continue;
            tma_load_4d(kdst + g * page_bytes, &k_map, bar, 0, 0, kvh, pages[g]);
            tma_load_4d(vdst + g * page_bytes, &v_map, bar, 0, 0, kvh, pages[g]);
          }
        }
        issued = j + 1;
      }
      if (*(volatile int*)&abort_s) {
        // wind down: let the copies in flight land before the CTA's shared memory is given up
        for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j) {
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&kv_full[j % STAGES]), (j / STAGES) & 1)) {
            if (globaltimer_ns() - t0 > 20000000ull) {  // 20 ms
              atomicCAS(&g_tc_error_word, 0, ERR_WAIT_DRAIN);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = instr_desc_bf16(QROWS, KT);
    constexpr uint32_t idesc_o = instr_desc_bf16(QROWS, HD) | INSTR_B_MN_MAJOR;
    bool ok = mbar_wait(smem_u32(&q_full), 0);
    if (!ok && lane == 0) atomicCAS(&g_tc_error_word, 0, ERR_WAIT_FULL);
    auto issue_s = [&](int j) {      // S(j) = Q K(j)^T into S buffer j & 1
      const int s = j % STAGES;
      if (!mbar_wait(smem_u32(&kv_full[s]), (j / STAGES) & 1)) {
        if (lane == 0) atomicCAS(&g_tc_error_word, 0, ERR_WAIT_FULL);
        ok = false;
        return;
      }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t kb = kv_s + s * STAGE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          mma_bf16(tmem_base + (j & 1) * KT, smem_desc_sw128(q_s + k * 32), smem_desc_sw128(kb + k * 32), idesc_s, k > 0);
        mma_commit(smem_u32(&s_ready[j & 1]));
      }
      __syncwarp();
    };
    if (ok) issue_s(0);
    if (ok && n_tiles > 1) issue_s(1);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (*(volatile int*)&abort_s) break;
      if (!mbar_wait(smem_u32(&p_ready[j & 1]), (j >> 1) & 1)) {
        if (lane == 0) atomicCAS(&g_tc_error_word, 0, ERR_WAIT_ACCUM);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int s = j % STAGES;
      const uint32_t vb = kv_s + s * STAGE_BYTES + K_BYTES;
      const int key0 = (tile_begin + j) * KT;
      if (key0 < lo || key0 + KT - 1 > hi) {
        // Value rows that no row may read hold whatever was there (a page that was not fetched,
        // the unwritten end of the last page): their probabilities are zero, but zero times a
        // stray NaN is not. Clear them.
        for (int row = lane; row < KT; row += 32) {
          const int key = key0 + row;
          if (key < lo || key > hi) {
#pragma unroll
            for (int c = 0; c < ROW_BYTES / 16; ++c) st_shared_v4(vb + row * ROW_BYTES + c * 16, 0u, 0u, 0u, 0u);
          }
        }
        fence_proxy_async();
        __syncwarp();
      }
      if (lane == 0) {
        const uint32_t pb = p_s + (j & 1) * P_BYTES;
#pragma unroll
        for (int ks = 0; ks < KT / 16; ++ks)
          mma_bf16(tmem_base + O_COL0 + (j & 1) * HD, smem_desc_sw128(pb + (ks >> 2) * (QROWS * 128) + (ks & 3) * 32),
                   smem_desc_sw128_mn(vb + ks * 16 * ROW_BYTES), idesc_o, ks > 0);
        mma_commit(smem_u32(&o_ready[j & 1]));
        mma_commit(smem_u32(&kv_empty[s]));     // keys and values of the stage have been read
      }
      __syncwarp();
      if (j + 2 < n_tiles) issue_s(j + 2);      // its S buffer was read in full before p_ready fired
    }
    if (!ok) abort_s = 1;
  } else {
    // -------------------------------------------------------------------- softmax warps
    const int quarter = warp & 3;                        // the TMEM lanes this warp may read
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int row_pos = row < nrows ? pos0 + row / p.g : -1;       // no key is valid for a padding row
    const int row_start = (row < nrows && p.window > 0) ? max(0, row_pos + 1 - p.window) : 0;
    const float scale_log2 = p.scale_log2;
    float o_acc[HD];
#pragma unroll
    for (int c = 0; c < HD; ++c) o_acc[c] = 0.f;
    float m = -INFINITY, l = 0.f, corr_saved = 0.f;      // m: running maximum of the raw dot products
    bool ok = true;

    auto fold = [&](int j) {        // o_acc = o_acc * corr_saved + O_tile(j)
      if (!mbar_wait(smem_u32(&o_ready[j & 1]), (j >> 1) & 1)) {
        if (lane == 0) atomicCAS(&g_tc_error_word, 0, ERR_WAIT_ACCUM);
        ok = false;
        return;
      }
      tc_fence_after_sync();
#pragma unroll
      for (int h = 0; h < HD / 32; ++h) {
        uint32_t v[32];
        tmem_ld_32(lane_addr + O_COL0 + (j & 1) * HD + h * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) o_acc[h * 32 + c] = fmaf(o_acc[h * 32 + c], corr_saved, __uint_as_float(v[c]));
      }
    };

    for (int j = 0; j < n_tiles; ++j) {
      if (*(volatile int*)&abort_s) { ok = false; break; }
      if (!mbar_wait(smem_u32(&s_ready[j & 1]), (j >> 1) & 1)) {
        if (lane == 0) atomicCAS(&g_tc_error_word, 0, ERR_WAIT_ACCUM);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      float s[KT];
#pragma unroll
      for (int h = 0; h < KT / 32; ++h) {
        uint32_t v[32];
        tmem_ld_32(lane_addr + (j & 1) * KT + h * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) s[h * 32 + c] = __uint_as_float(v[c]);
      }
      const int key0 = (tile_begin + j) * KT;
      // a tile needs no mask if it lies wholly before the first row's position and inside the
      // last row's window
      const bool full = key0 + KT - 1 <= pos0 && (p.window <= 0 || key0 >= hi + 1 - p.window);
      if (!full) {
#pragma unroll
        for (int c = 0; c < KT; ++c)
          if (!(key0 + c >= row_start && key0 + c <= row_pos)) s[c] = -INFINITY;
      }
      float m_new = m;
#pragma unroll
      for (int c = 0; c < KT; ++c) m_new = fmaxf(m_new, s[c]);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;          // nothing valid yet: avoid inf - inf
      const float corr = m == -INFINITY ? 0.f : fast_exp2((m - m_use) * scale_log2);
      const float neg_m = -m_use * scale_log2;
      m = m_new;
      float l_add = 0.f;
      const uint32_t prow = p_s + (j & 1) * P_BYTES + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < KT / 8; ++c8) {
        float pr[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pr[e] = fast_exp2(fmaf(s[c8 * 8 + e], scale_log2, neg_m));   // exp2(-inf) = 0 for masked keys
          l_add += pr[e];
        }
        // block of 64 keys c8 / 8, 16-byte chunk c8 % 8 of the row, swizzled with the row
        st_shared_v4(prow + (c8 >> 3) * (QROWS * 128) + (((c8 & 7) ^ (row & 7)) << 4), pack_bf16(pr[0], pr[1]),
                     pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
      }
      l = l * corr + l_add;
      fence_proxy_async();            // the tensor core reads P through the async proxy
      tc_fence_before_sync();         // this thread's reads of S are over
      mbar_arrive(smem_u32(&p_ready[j & 1]));
      if (j > 0) {
        fold(j - 1);
        if (!ok) break;
      }
      corr_saved = corr;
    }
    if (ok && n_tiles > 0) fold(n_tiles - 1);
    if (ok && row < nrows) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(q_begin + tok0 + row / p.g) * p.Hq + kvh * p.g + row % p.g) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        uint4 w;
        w.x = pack_bf16(o_acc[c] * inv, o_acc[c + 1] * inv);
        w.y = pack_bf16(o_acc[c + 2] * inv, o_acc[c + 3] * inv);
        w.z = pack_bf16(o_acc[c + 4] * inv, o_acc[c + 5] * inv);
        w.w = pack_bf16(o_acc[c + 6] * inv, o_acc[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = w;
      }
    }
    if (!ok) abort_s = 1;
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
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tile_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return gb::fail(GB_CUDA_ERROR, "attention_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((max_q_len + tokens_per_tile - 1) / tokens_per_tile, p.Hkv, R);
  return gb::check_pdl_launch(gb::launch_pdl(attention_tile_tc_kernel, grid, dim3(THREADS), SMEM_BYTES, stream,
                                             dim3(1, 1, 1), qm, km, vm, p),
                              "attention_tc (tile)");
}

int tile_tc_error_check() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error_word, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_tc_error_word, &zero, sizeof(int));
  }
  return v;
}

}  // namespace attn

#else  // other head sizes: the mma.sync kernels

namespace attn {
bool tile_tc_takes(const Params&, int, long long) { return false; }
int launch_tile_tc(const Params&, int, long long, int, int, cudaStream_t) {
  return gb::fail(GB_UNSUPPORTED, "attention_tc: head size %d", GB_HEAD_DIM);
}
int tile_tc_error_check() { return 0; }
}  // namespace attn

#endif
