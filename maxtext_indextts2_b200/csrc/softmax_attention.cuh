// Causal softmax attention with grouped key heads and rotary positions, over the paged cache and a ragged batch.
//
// For the query row at position i of page group s and query head h (key head g = h / (H / G)):
//
//   s(j)  = scale * <rot(q_h, i), rot(k_g(j), j)>        for lo <= j <= i, lo = max(0, i - window + 1) (window 0: lo = 0)
//   p(j)  = exp(s(j) - max_j s) / sum_j exp(s(j) - max_j s)
//   out_h = out_scale * sum_j p(j) v_g(j)
//
// rot(t, p) turns the channel pairs (2c, 2c + 1), c < rot_dims / 2, of a head by the angle p * rot_freq[c] (fp32 angle, fp32
// sine and cosine); the remaining channels pass.  A design whose values are the un-rotated keys (values_are_keys) gets the key
// projection written twice: rotated into the key pool, as projected into the value pool.
//
//   rope_append_kernel         per row: bias already in the projection; rotates q and k, writes q, appends k and v to the pages
//   softmax_attention_rows_kernel<T>   one CTA per (query tile of <= 16 rows of one sequence, query head); keys walked in tiles
//                              staged as fp32 in shared memory; running maximum and sum per row; everything fp32 (T is only the
//                              dtype of q, the pools and the output).  Serves float32 engines, every geometry, and decode rows.
//   softmax_attention_mma_kernel       bf16: the same work item on mma.sync m16n8k16 (S = Q K^T and O += P V), for dim and vdim
//                              that are multiples of 16.
#pragma once

#include "common.cuh"
#include "layer_ops.cuh"
#include "linear_any.cuh"

namespace mtx {

template <typename T>
struct RopeAppendArgs {
  const float* proj;     // [rows, ld]: q at column q_col, k at k_col, v at v_col (v_col < 0: the values are the keys)
  long long ld;
  int q_col, k_col, v_col;
  const float* rot_freq;  // [rot_dims / 2]
  T* q_out;               // [rows, H * d]
  T* k_pages;
  T* v_pages;
  const int* group;
  const int* pos;
  const int* page_map;
  int heads, kv_heads, dim, vdim, rot_dims;
  int num_pages, tokens_per_page, max_pages;
};

template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim, half = d / 2, rh = a.rot_dims / 2;
  const float* row = a.proj + size_t(r) * a.ld;
  const int p = a.pos[r], grp = a.group[r];
  const size_t slot = size_t(a.page_map[size_t(grp) * a.max_pages + p / a.tokens_per_page]) * a.tokens_per_page + p % a.tokens_per_page;
  const float fp = float(p);
  // pairs of q and of k: unit u = (head, pair)
  const int q_pairs = H * half, k_pairs = G * half;
  for (int u = tid; u < q_pairs + k_pairs; u += blockDim.x) {
    const bool is_q = u < q_pairs;
    const int v = is_q ? u : u - q_pairs, head = v / half, c = v % half;
    const float* src = row + (is_q ? a.q_col : a.k_col) + head * d + 2 * c;
    float x0 = src[0], x1 = src[1];
    if (c < rh) {
      float sn, cs;
      sincosf(fp * a.rot_freq[c], &sn, &cs);
      const float y0 = x0 * cs - x1 * sn, y1 = x1 * cs + x0 * sn;
      x0 = y0;
      x1 = y1;
    }
    T* dst = is_q ? a.q_out + size_t(r) * H * d + head * d + 2 * c
                  : a.k_pages + (size_t(head) * a.num_pages * a.tokens_per_page + slot) * d + 2 * c;
    dst[0] = to_act<T>(x0);
    dst[1] = to_act<T>(x1);
  }
  if (d & 1) {  // an odd last channel is never rotated
    for (int u = tid; u < H + G; u += blockDim.x) {
      const bool is_q = u < H;
      const int head = is_q ? u : u - H;
      const float x = row[(is_q ? a.q_col : a.k_col) + head * d + d - 1];
      if (is_q) a.q_out[size_t(r) * H * d + head * d + d - 1] = to_act<T>(x);
      else a.k_pages[(size_t(head) * a.num_pages * a.tokens_per_page + slot) * d + d - 1] = to_act<T>(x);
    }
  }
  const int vsrc = a.v_col < 0 ? a.k_col : a.v_col;
  for (int e = tid; e < G * dv; e += blockDim.x) {
    const int kv = e / dv, c = e % dv;
    a.v_pages[(size_t(kv) * a.num_pages * a.tokens_per_page + slot) * dv + c] = to_act<T>(row[vsrc + e]);
  }
}

template <typename T>
struct SoftmaxAttnArgs {
  const T* q;            // [rows, H * d]
  T* out;                // [rows, ld_out]; head h writes columns [h * dv, (h + 1) * dv)
  long long ld_out;
  const T* k_pages;
  const T* v_pages;
  const int* group;
  const int* pos;
  const int* page_map;
  const int* tile_row0;  // [n_tiles + 1]
  int heads, kv_heads, dim, vdim, window;
  int num_pages, tokens_per_page, max_pages;
  float scale, out_scale;
};

constexpr int kSmaxThreads = 256, kSmaxRows = 16, kSmaxKeys = 32;
constexpr int kSmaxMaxAcc = 32;  // kSmaxRows * vdim <= kSmaxThreads * kSmaxMaxAcc: vdim <= 512

inline size_t softmax_attn_smem_bytes(int dim, int vdim) {
  return sizeof(float) * (size_t(kSmaxRows) * dim + size_t(kSmaxKeys) * (dim + 1) + size_t(kSmaxKeys) * vdim + size_t(kSmaxRows) * kSmaxKeys +
                          3 * kSmaxRows);
}

template <typename T>
__global__ void __launch_bounds__(kSmaxThreads) softmax_attention_rows_kernel(const SoftmaxAttnArgs<T> a) {
  extern __shared__ float smem[];
  const int d = a.dim, dv = a.vdim, rep = a.heads / a.kv_heads;
  float* sq = smem;                        // [16][d]
  float* sk = sq + kSmaxRows * d;          // [32][d + 1]
  float* sv = sk + kSmaxKeys * (d + 1);    // [32][dv]
  float* sp = sv + kSmaxKeys * dv;         // [16][32]
  float* s_max = sp + kSmaxRows * kSmaxKeys;  // [16] running maximum
  float* s_sum = s_max + kSmaxRows;           // [16] running sum
  float* s_fix = s_sum + kSmaxRows;           // [16] factor that brings the old accumulators to the new maximum
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  griddep_wait();
  const int r0 = a.tile_row0[blockIdx.x], nr = a.tile_row0[blockIdx.x + 1] - r0, h = blockIdx.y, g = h / rep;
  const int p0 = a.pos[r0], grp = a.group[r0];  // row r0 + i has position p0 + i
  const int p_last = p0 + nr - 1;
  int lo = 0;
  if (a.window > 0 && p0 - a.window + 1 > 0) lo = p0 - a.window + 1;
  for (int e = tid; e < nr * d; e += kSmaxThreads) sq[e] = act_f32(a.q[size_t(r0 + e / d) * a.heads * d + h * d + e % d]) * a.scale;
  if (tid < kSmaxRows) {
    s_max[tid] = -INFINITY;
    s_sum[tid] = 0.0f;
  }
  float acc[kSmaxMaxAcc];
#pragma unroll
  for (int u = 0; u < kSmaxMaxAcc; ++u) acc[u] = 0.0f;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;
  const size_t head_rows = size_t(g) * a.num_pages * a.tokens_per_page;
  for (int j0 = lo; j0 <= p_last; j0 += kSmaxKeys) {
    const int nk = p_last - j0 + 1 < kSmaxKeys ? p_last - j0 + 1 : kSmaxKeys;
    __syncthreads();
    for (int e = tid; e < nk * d; e += kSmaxThreads) {
      const int jj = e / d, c = e % d, j = j0 + jj;
      const size_t row = head_rows + size_t(pages[j / a.tokens_per_page]) * a.tokens_per_page + j % a.tokens_per_page;
      sk[jj * (d + 1) + c] = act_f32(a.k_pages[row * d + c]);
    }
    for (int e = tid; e < nk * dv; e += kSmaxThreads) {
      const int jj = e / dv, c = e % dv, j = j0 + jj;
      const size_t row = head_rows + size_t(pages[j / a.tokens_per_page]) * a.tokens_per_page + j % a.tokens_per_page;
      sv[jj * dv + c] = act_f32(a.v_pages[row * dv + c]);
    }
    __syncthreads();
    for (int e = tid; e < nr * kSmaxKeys; e += kSmaxThreads) {
      const int i = e / kSmaxKeys, jj = e % kSmaxKeys, j = j0 + jj, pi = p0 + i;
      float s = -INFINITY;
      if (jj < nk && j <= pi && (a.window <= 0 || pi - j < a.window)) {
        const float* qv = sq + i * d;
        const float* kv = sk + jj * (d + 1);
        s = 0.0f;
        for (int c = 0; c < d; ++c) s = fmaf(qv[c], kv[c], s);
      }
      sp[e] = s;
    }
    __syncthreads();
    for (int i = warp; i < nr; i += kSmaxThreads / 32) {  // kSmaxKeys == 32: one key per lane
      const float s = sp[i * kSmaxKeys + lane];
      float m = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float m_old = s_max[i], m_new = fmaxf(m_old, m);
      const float p = (m_new == -INFINITY || s == -INFINITY) ? 0.0f : expf(s - m_new);
      const float fix = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
      const float sum = warp_sum(p);
      sp[i * kSmaxKeys + lane] = p;
      if (lane == 0) {
        s_max[i] = m_new;
        s_sum[i] = s_sum[i] * fix + sum;
        s_fix[i] = fix;
      }
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kSmaxMaxAcc; ++u) {
      const int o = tid + u * kSmaxThreads;
      if (o < nr * dv) {
        const int i = o / dv, c = o % dv;
        const float* pv = sp + i * kSmaxKeys;
        float s = acc[u] * s_fix[i];
        for (int jj = 0; jj < nk; ++jj) s = fmaf(pv[jj], sv[jj * dv + c], s);
        acc[u] = s;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < kSmaxMaxAcc; ++u) {
    const int o = tid + u * kSmaxThreads;
    if (o < nr * dv) {
      const int i = o / dv, c = o % dv;
      a.out[size_t(r0 + i) * a.ld_out + h * dv + c] = to_act<T>(acc[u] * a.out_scale / s_sum[i]);
    }
  }
}

}  // namespace mtx
