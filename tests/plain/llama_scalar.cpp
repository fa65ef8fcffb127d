// A second plain restatement of the reference's dense Llama decoder, in scalar C++: one token at a
// time, keys and values appended to a growing array per layer, every sum taken sequentially in
// 32-bit, as the reference's CPU code takes them. It exists to cross-check the numpy restatement
// (llama_plain.py), which works on whole sequences with numpy's own summation order: the two were
// written apart, from the same cited lines, and must agree to rounding. Like that file it rests on
// the formulas (the reference is Rust and cannot be built without a Rust toolchain), shares no code
// with garuda_b200, and is compiled by the tests alone
// (g++ -O2 -ffp-contract=off: no fused multiply-adds, which the reference's code does not use).
#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

namespace {

struct Sizes {
  int32_t layers, width, heads, kv_heads, head_dim, inner, vocab;
  int32_t interleaved;   // rotation pairs (2i, 2i + 1), else (i, i + head_dim / 2)
  int32_t tied;          // the head is the embedding table
  float eps, theta;
};

// garuda/src/simd/mod.rs:13-16: products summed left to right.
float dot(const float* a, const float* b, int n) {
  float s = 0.0f;
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

// garuda/src/simd/mod.rs:72-86: out[r] = dot(row r, x) for a row-major [rows, cols] matrix.
void matvec(const float* m, int rows, int cols, const float* x, float* out) {
  for (int r = 0; r < rows; ++r) out[r] = dot(m + static_cast<size_t>(r) * cols, x, cols);
}

// garuda/src/simd/mod.rs:166-173 then garuda/src/llama/mod.rs:733-738: the mean of squares with eps
// inside the root, the scale applied first, the weight second.
void norm(const float* x, const float* weight, int n, float eps, float* out) {
  float sq = 0.0f;
  for (int i = 0; i < n; ++i) sq += x[i] * x[i];
  const float mean_sq = sq / static_cast<float>(n);
  const float scale = 1.0f / std::sqrt(mean_sq + eps);
  for (int i = 0; i < n; ++i) out[i] = x[i] * scale;
  for (int i = 0; i < n; ++i) out[i] *= weight[i];
}

// garuda/src/simd/mod.rs:196-206: pair i is rotated by pos * theta^(-2i / head_dim), frequency,
// angle, sine and cosine in 32-bit. The reference pairs (2i, 2i + 1); for the unpermuted rows of
// a safetensors folder the same rotation pairs (i, i + head_dim / 2).
void rotate(float* v, int head_dim, int pos, float theta, bool interleaved) {
  const int half = head_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float freq = 1.0f / std::pow(theta, 2.0f * static_cast<float>(i) / static_cast<float>(head_dim));
    const float angle = static_cast<float>(pos) * freq;
    const float sn = std::sin(angle), cs = std::cos(angle);
    const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
    const float a = v[ia], b = v[ib];
    v[ia] = a * cs - b * sn;
    v[ib] = a * sn + b * cs;
  }
}

// garuda/src/simd/mod.rs:132-158: the maximum taken out, exponentials summed in order, one
// reciprocal; uniform when the maximum or the sum is no number to divide by.
void softmax(std::vector<float>& x) {
  if (x.empty()) return;
  float mx = -std::numeric_limits<float>::infinity();
  for (float v : x) mx = std::fmax(mx, v);
  const float uniform = 1.0f / static_cast<float>(x.size());
  if (!std::isfinite(mx)) {
    for (float& v : x) v = uniform;
    return;
  }
  float sum = 0.0f;
  for (float& v : x) {
    v = std::exp(v - mx);
    sum += v;
  }
  if (std::isfinite(sum) && sum > 0.0f) {
    const float inv = 1.0f / sum;
    for (float& v : x) v *= inv;
    return;
  }
  for (float& v : x) v = uniform;
}

}  // namespace

// tensors: the embedding table; for every layer the input norm, q, k, v and o projections, the
// post-attention norm, gate, up and down projections; the final norm; the head (unused when tied).
// windows[layer]: positions a query looks back over, itself included; 0: all of them.
// logits: [T, vocab]. Returns 0, or 1 for a token outside the vocabulary (refused before any layer
// runs: garuda/src/llama/mod.rs:1078-1085).
extern "C" int llama_scalar_forward(const Sizes* sizes, const float* const* tensors, const int32_t* windows,
                                    const int32_t* tokens, int32_t T, float* logits) {
  const Sizes c = *sizes;
  const int d = c.width, hd = c.head_dim, q_dim = c.heads * hd, kv_dim = c.kv_heads * hd;
  for (int t = 0; t < T; ++t)
    if (tokens[t] < 0 || tokens[t] >= c.vocab) return 1;
  const float* embedding = tensors[0];
  const float* final_norm = tensors[1 + 9 * c.layers];
  const float* head = c.tied ? embedding : tensors[2 + 9 * c.layers];
  // the cache: per layer, the rotated keys and the values of every position so far
  std::vector<std::vector<float>> keys(c.layers), values(c.layers);
  std::vector<float> x(d), h(d), q(q_dim), k(kv_dim), v(kv_dim), context(q_dim), a(d), g(c.inner), u(c.inner), y(d);
  const int group = c.heads / c.kv_heads;                  // garuda/src/llama/mod.rs:781
  const float scale = 1.0f / std::sqrt(static_cast<float>(hd));   // :797
  for (int t = 0; t < T; ++t) {
    const float* row = embedding + static_cast<size_t>(tokens[t]) * d;   // :198-200, no scaling
    for (int i = 0; i < d; ++i) x[i] = row[i];
    for (int l = 0; l < c.layers; ++l) {
      const float* const* w = tensors + 1 + 9 * l;
      // garuda/src/llama/mod.rs:862-880: norm, projections, attention, output projection, residual
      norm(x.data(), w[0], d, c.eps, h.data());
      matvec(w[1], q_dim, d, h.data(), q.data());
      matvec(w[2], kv_dim, d, h.data(), k.data());
      matvec(w[3], kv_dim, d, h.data(), v.data());
      const int pos = static_cast<int>(keys[l].size()) / kv_dim;       // :783: the cache's own length
      for (int hh = 0; hh < c.heads; ++hh) rotate(q.data() + hh * hd, hd, pos, c.theta, c.interleaved != 0);
      for (int hh = 0; hh < c.kv_heads; ++hh) rotate(k.data() + hh * hd, hd, pos, c.theta, c.interleaved != 0);
      keys[l].insert(keys[l].end(), k.begin(), k.end());               // :791: the rotated key is what is kept
      values[l].insert(values[l].end(), v.begin(), v.end());
      // garuda/src/cache/mod.rs:333-338, read after the append: the last `window` positions
      const int end = pos + 1;
      const int start = windows[l] > 0 && end > windows[l] ? end - windows[l] : 0;
      for (int i = 0; i < q_dim; ++i) context[i] = 0.0f;
      for (int hh = 0; hh < c.heads; ++hh) {                           // :793-818
        const float* q_h = q.data() + hh * hd;
        const int at = (hh / group) * hd;
        std::vector<float> scores;
        for (int j = start; j < end; ++j)
          scores.push_back(dot(q_h, keys[l].data() + static_cast<size_t>(j) * kv_dim + at, hd) * scale);
        softmax(scores);
        float* out_h = context.data() + hh * hd;
        for (int j = start; j < end; ++j) {
          const float p = scores[j - start];
          const float* val = values[l].data() + static_cast<size_t>(j) * kv_dim + at;
          for (int ch = 0; ch < hd; ++ch) out_h[ch] += val[ch] * p;     // simd/mod.rs:183-186
        }
      }
      matvec(w[4], d, q_dim, context.data(), a.data());
      for (int i = 0; i < d; ++i) x[i] += a[i];
      // garuda/src/llama/mod.rs:885 and :1002-1020: norm, gate and up, SiLU on the gate, times up, down
      norm(x.data(), w[5], d, c.eps, h.data());
      matvec(w[6], c.inner, d, h.data(), g.data());
      matvec(w[7], c.inner, d, h.data(), u.data());
      for (int i = 0; i < c.inner; ++i) g[i] /= 1.0f + std::exp(-g[i]);   // simd/mod.rs:161-163
      for (int i = 0; i < c.inner; ++i) g[i] *= u[i];
      matvec(w[8], d, c.inner, g.data(), y.data());
      for (int i = 0; i < d; ++i) x[i] += y[i];
    }
    // garuda/src/llama/mod.rs:1110-1113 and :1238-1240: the final norm, then the head
    norm(x.data(), final_norm, d, c.eps, h.data());
    matvec(head, c.vocab, d, h.data(), logits + static_cast<size_t>(t) * c.vocab);
  }
  return 0;
}
