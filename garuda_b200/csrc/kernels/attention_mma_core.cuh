// What the mma.sync attention kernels of one head size share: fragment loads, the m16n8k16 product,
// a warp's running softmax state, and one tile of 64 keys for a warp's 16 query rows.
//
// garuda/src/llama/mod.rs:793-818: s_j = dot(q, K_j) * scale, softmax with the maximum subtracted,
// sum of p_j V_j, everything but the operands of the two products in 32-bit.
#pragma once

#include <cuda_bf16.h>

#include <cstdint>

namespace attn_mma {

constexpr int KT = 64;              // keys per tile

// Where a tile's rows lie in shared memory. Padded: rows of LD elements one after the other (what the
// per-thread copies write). Swizzled: what TMA writes with the 128-byte swizzle: 64-element halves of
// the head one after the other, each [64 keys][128 bytes] with a row's 16-byte chunks XORed with the
// row's low three bits (the half's base is 1024-byte aligned).
template <int HD, int LD>
struct PaddedTile {
  const __nv_bfloat16* base;
  __device__ __forceinline__ const void* chunk(int key, int c) const { return base + key * LD + c * 8; }
};
template <int HD, int KEYS>
struct SwizzledTile {
  const uint8_t* base;
  __device__ __forceinline__ const void* chunk(int key, int c) const {
    return base + (c >> 3) * (KEYS * 128) + key * 128 + (((c & 7) ^ (key & 7)) << 4);
  }
};

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
// 2^x on the special-function unit (about 2^-22 relative error; the result feeds a bfloat16 operand
// and 32-bit sums). -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One warp's running state over the keys it has seen: 16 query rows, of which a thread holds the
// two rows lane / 4 and lane / 4 + 8.
template <int HD>
struct WarpState {
  float o[HD / 8][4];
  float m[2], l[2];
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

// One tile of 64 keys for one warp's 16 rows: S = Q K^T, scale and mask, running softmax in
// 32-bit, O += P V. qf: the warp's query fragments; key0: position of the tile's first key;
// row_pos / row_start: last and first key each of the thread's two rows may read; full: every key
// of the tile is inside every row's range (no mask needed). The running maximum st.m is kept
// unscaled (a raw dot product); the merges scale it.
// KEYS: keys in the tile (64, or 32 for the smaller tiles of the decode kernel that copies by TMA).
template <int HD, typename Tile, int KEYS = KT>
__device__ __forceinline__ void process_tile(WarpState<HD>& st, const uint32_t (&qf)[HD / 16][4],
                                             const Tile ks, const Tile vs, int key0,
                                             const int (&row_pos)[2], const int (&row_start)[2], float scale_log2,
                                             bool full) {
  const int lane = threadIdx.x & 31;
  float s[KEYS / 8][4];
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
    for (int n2 = 0; n2 < KEYS / 16; ++n2) {
      uint32_t b[4];
      const int key = n2 * 16 + (lane % 8) + (lane / 16) * 8;
      ldmatrix_x4(b, ks.chunk(key, kk * 2 + ((lane / 8) % 2)));
      mma_16816(s[2 * n2], qf[kk], b[0], b[1]);
      mma_16816(s[2 * n2 + 1], qf[kk], b[2], b[3]);
    }
  }
  // Mask (only where the tile is not wholly inside every row's range), then the running maximum of
  // the raw dot products: the scale is positive, so it can wait until the exponent, where
  // exp2(s * scale_log2 - m * scale_log2) is one multiply-add and one special-function op.
  float m_new[2] = {st.m[0], st.m[1]};
  if (!full) {
#pragma unroll
    for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = key0 + n * 8 + (lane % 4) * 2 + (e & 1);
        if (!(j >= row_start[i] && j <= row_pos[i])) s[n][e] = -INFINITY;
      }
  }
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], s[n][e]);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
    m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
  }
  float corr[2], neg_m[2], l_add[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float m_use = m_new[i] == -INFINITY ? 0.f : m_new[i];     // nothing valid yet: avoid inf - inf
    corr[i] = st.m[i] == -INFINITY ? 0.f : fast_exp2((st.m[i] - m_use) * scale_log2);
    neg_m[i] = -m_use * scale_log2;
    st.m[i] = m_new[i];
  }
  uint32_t pf[KEYS / 16][4];
#pragma unroll
  for (int n = 0; n < KEYS / 8; ++n) {
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      pr[e] = fast_exp2(fmaf(s[n][e], scale_log2, neg_m[e >> 1]));   // exp2(-inf) = 0 for masked keys
      l_add[e >> 1] += pr[e];
    }
    pf[n / 2][(n % 2) * 2 + 0] = pack_bf16(pr[0], pr[1]);
    pf[n / 2][(n % 2) * 2 + 1] = pack_bf16(pr[2], pr[3]);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) st.l[i] = st.l[i] * corr[i] + l_add[i];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    st.o[n][0] *= corr[0]; st.o[n][1] *= corr[0];
    st.o[n][2] *= corr[1]; st.o[n][3] *= corr[1];
  }
#pragma unroll
  for (int kk = 0; kk < KEYS / 16; ++kk) {
#pragma unroll
    for (int n2 = 0; n2 < HD / 16; ++n2) {
      uint32_t b[4];
      const int key = kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
      ldmatrix_x4_trans(b, vs.chunk(key, n2 * 2 + (lane / 16)));
      mma_16816(st.o[2 * n2], pf[kk], b[0], b[1]);
      mma_16816(st.o[2 * n2 + 1], pf[kk], b[2], b[3]);
    }
  }
}


}  // namespace attn_mma
