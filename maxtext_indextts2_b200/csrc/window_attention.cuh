// Sliding-window attention with independent (sigmoid) key weights, a bias by distance, and mixing of the heads' weights,
// over a paged cache and a ragged batch.
//
// For the query row at position i of page group s, every key j with 0 <= i - j < window gets, per query head g,
//
//   s_g(j)  = cap * tanh(scale * <q_g, k_kv(g)(j)> / cap) + dist_bias[i - j, g]      (cap = 0: no soft cap)
//   w_g(j)  = 1 / (1 + exp(-(s_g(j) + head_bias[g])))                                (no normalisation over the keys)
//   w'_h(j) = sum_g talk[h, g] * w_g(j)                                              (talk = identity when null)
//   out_h   = sum_j w'_h(j) * v_kv(h)(j)
//
// all in fp32.  `dist_bias` is a table over the distance itself ([window, H]): a design that buckets distances expands its
// buckets into it at load time, so the kernel has no opinion about the bucket rule.  Rows are independent: a prompt portion is a
// run of rows with consecutive positions, a decoded token a single row, and both sit in one launch.  The keys and values of the
// rows of this step are in the cache already (the projection's post-kernel appends them before this kernel starts).
//
// window_attention_rows_kernel: one CTA per row, all heads (the mixing needs every head's weight of a (row, key) pair).  Keys are
// walked in tiles of `kt` keys staged in shared memory as fp32; (head, key) pairs are spread over the threads for the scores,
// (head, value column) pairs for the products.  Serves decode rows, float32 engines and any head geometry.
#pragma once

#include "common.cuh"
#include "linear_any.cuh"

namespace mtx {

template <typename T>
struct WindowAttnArgs {
  const T* q;            // [rows, H * d]
  T* out;                // [rows, H * dv]
  const T* k_pages;      // [G, num_pages, tokens_per_page, d]
  const T* v_pages;      // [G, num_pages, tokens_per_page, dv]
  const int* group;      // [rows]
  const int* pos;        // [rows]
  const int* page_map;   // [groups, max_pages]
  const float* dist_bias;  // [window, H]
  const float* head_bias;  // [H] or null
  const float* talk;       // [H, H] or null
  int rows, heads, kv_heads, dim, vdim, window;
  int num_pages, tokens_per_page, max_pages;
  int kt;  // keys per tile
  float scale, softcap;
};

constexpr int kWinThreads = 256;
constexpr int kWinMaxAcc = 8;  // output elements per thread: H * dv <= kWinThreads * kWinMaxAcc

inline size_t window_attn_smem_bytes(int heads, int kv_heads, int dim, int vdim, int kt) {
  return sizeof(float) * (size_t(heads) * dim + size_t(kv_heads) * kt * (dim + 1) + size_t(kv_heads) * kt * vdim + 2 * size_t(heads) * kt +
                          size_t(heads) * heads + heads);
}

template <typename T>
__global__ void __launch_bounds__(kWinThreads) window_attention_rows_kernel(const WindowAttnArgs<T> a) {
  extern __shared__ float smem[];
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim, KT = a.kt, rep = H / G;
  float* sq = smem;                       // [H][d]
  float* sk = sq + H * d;                 // [G][KT][d + 1]
  float* sv = sk + G * KT * (d + 1);      // [G][KT][dv]
  float* sw = sv + G * KT * dv;           // [H][KT] raw weights
  float* sm = sw + H * KT;                // [H][KT] mixed weights
  float* stalk = sm + H * KT;             // [H][H]
  float* spb = stalk + H * H;             // [H]
  const int tid = threadIdx.x, r = blockIdx.x;
  griddep_wait();
  const int i = a.pos[r], grp = a.group[r];
  const int lo = i - a.window + 1 > 0 ? i - a.window + 1 : 0;
  for (int e = tid; e < H * d; e += kWinThreads) sq[e] = act_f32(a.q[size_t(r) * H * d + e]);
  for (int e = tid; e < H * H; e += kWinThreads) stalk[e] = a.talk ? a.talk[e] : ((e / H == e % H) ? 1.0f : 0.0f);
  for (int e = tid; e < H; e += kWinThreads) spb[e] = a.head_bias ? a.head_bias[e] : 0.0f;
  float acc[kWinMaxAcc];
#pragma unroll
  for (int u = 0; u < kWinMaxAcc; ++u) acc[u] = 0.0f;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;
  for (int j0 = lo; j0 <= i; j0 += KT) {
    const int nk = i - j0 + 1 < KT ? i - j0 + 1 : KT;
    __syncthreads();  // the previous tile's products are done (and, first time, the staging above is visible)
    for (int e = tid; e < G * nk * d; e += kWinThreads) {
      const int c = e % d, jj = (e / d) % nk, kv = e / (d * nk);
      const int j = j0 + jj;
      const size_t row = (size_t(kv) * a.num_pages + pages[j / a.tokens_per_page]) * a.tokens_per_page + j % a.tokens_per_page;
      sk[(kv * KT + jj) * (d + 1) + c] = act_f32(a.k_pages[row * d + c]);
    }
    for (int e = tid; e < G * nk * dv; e += kWinThreads) {
      const int c = e % dv, jj = (e / dv) % nk, kv = e / (dv * nk);
      const int j = j0 + jj;
      const size_t row = (size_t(kv) * a.num_pages + pages[j / a.tokens_per_page]) * a.tokens_per_page + j % a.tokens_per_page;
      sv[(kv * KT + jj) * dv + c] = act_f32(a.v_pages[row * dv + c]);
    }
    __syncthreads();
    for (int e = tid; e < H * nk; e += kWinThreads) {
      const int jj = e % nk, g = e / nk;
      const float* qv = sq + g * d;
      const float* kvp = sk + ((g / rep) * KT + jj) * (d + 1);
      float s = 0.0f;
      for (int c = 0; c < d; ++c) s = fmaf(qv[c], kvp[c], s);
      s *= a.scale;
      if (a.softcap > 0.0f) s = a.softcap * tanhf(s / a.softcap);
      s += a.dist_bias[size_t(i - (j0 + jj)) * H + g] + spb[g];
      sw[g * KT + jj] = 1.0f / (1.0f + expf(-s));
    }
    __syncthreads();
    for (int e = tid; e < H * nk; e += kWinThreads) {
      const int jj = e % nk, h = e / nk;
      float m = 0.0f;
      for (int g = 0; g < H; ++g) m = fmaf(stalk[h * H + g], sw[g * KT + jj], m);
      sm[h * KT + jj] = m;
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kWinMaxAcc; ++u) {
      const int o = tid + u * kWinThreads;
      if (o < H * dv) {
        const int h = o / dv, c = o % dv;
        const float* wv = sm + h * KT;
        const float* vv = sv + (h / rep) * KT * dv + c;
        float s = acc[u];
        for (int jj = 0; jj < nk; ++jj) s = fmaf(wv[jj], vv[jj * dv], s);
        acc[u] = s;
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kWinMaxAcc; ++u) {
    const int o = tid + u * kWinThreads;
    if (o < H * dv) a.out[size_t(r) * H * dv + o] = to_act<T>(acc[u]);
  }
}

}  // namespace mtx
