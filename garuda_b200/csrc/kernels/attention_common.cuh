// What the attention kernels of one library share: the argument block and the hand-over from the
// general entry point to the tcgen05 kernel for prompt portions.
#pragma once

#include "common.cuh"

namespace attn {

constexpr int ROWS_DECODE = 16;     // a request with at most this many (token, head-of-group) rows is a decode request

struct Params {
  const __nv_bfloat16* q;        // [T, Hq, HD]
  const __nv_bfloat16* k_pool;   // [pages, Hkv, page_size, HD]
  const __nv_bfloat16* v_pool;
  __nv_bfloat16* out;            // [T, Hq * HD]
  const int32_t* block_table;    // [R, table_width]
  const int32_t* cu_q;           // [R + 1]
  const int32_t* kv_lens;        // [R]
  int table_width, Hq, Hkv, g, window, page_size;
  float scale_log2;              // scale * log2(e)
};

// True if the tcgen05 kernel takes this shape (head size 64 or 128, a power-of-two group, pages of
// a multiple of 8 keys that divide 128).
bool tile_tc_takes(const Params& p, int T, long long pages);
// Launches it for every request with more than ROWS_DECODE rows. Returns a GbStatus.
int launch_tile_tc(const Params& p, int T, long long pages, int R, int max_q_len, cudaStream_t stream);
// Non-zero if one of its CTAs gave up on a wait since the last call; clears it.
int tile_tc_error_check();
// Its kernels' failed waits also write their code to this word of pinned host memory (null: none).
int tile_tc_set_error_sink(int* host_word);

// The decode kernel that brings keys and values in by TMA (attention_decode_tma.cu; head sizes 64 and
// 128, pages of 8 to 128 keys). `ranks`: CTAs that share one request's keys, as a thread-block cluster
// (`cluster`) or independently; more than one independent CTA need `decode_tma_scratch_bytes` of
// scratch whose first 64 KB are zero before the first launch.
bool decode_tma_takes(const Params& p, long long pages);
int decode_tma_max_ranks(bool cluster);
long long decode_tma_scratch_bytes(int R, int kv_heads, int ranks);
int launch_decode_tma(const Params& p, long long pages, int R, int ranks, bool cluster, void* scratch,
                      long long scratch_bytes, cudaStream_t stream);
int decode_tma_error_check();
int decode_tma_set_error_sink(int* host_word);

}  // namespace attn
