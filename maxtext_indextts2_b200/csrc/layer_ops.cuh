// Row-wise steps of a layered model between its matrix products, for a ragged batch (every row = one token of some sequence):
//
//   embed_rows_kernel       x = embedding[token] * scale (fp32 residual) and its copy in the matmul dtype
//   qkv_post_kernel         per-head RMS norm of q and k (a weight vector shared by the heads), mixing of the values with the
//                           values an earlier layer computed for the same token, append of k and v to the paged cache
//   norm_residual_kernel    x += gain * y / sqrt(mean(y^2) + eps)   (a normalisation with ONE gain, on the sublayer's OUTPUT)
//   scalar_norm_rows_kernel n = gain * x[row] / sqrt(mean(x[row]^2) + eps) for a gathered subset of rows (before the logits)
//
// Everything here is fp32 arithmetic; T is the dtype the matrix products and the cache use (bf16, or float for a float32 engine).
#pragma once

#include "common.cuh"
#include "linear_any.cuh"

namespace mtx {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// sum over the block; every thread gets the result.  `red` holds one float per warp.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = 0.0f;
  for (int w = 0; w < nw; ++w) r += red[w];  // fixed order
  return r;
}

template <typename T>
__global__ void embed_rows_kernel(const int* token, const T* embedding, int vocab, float scale, float* x, T* xa, int width) {
  griddep_wait();
  const int r = blockIdx.x;
  int tok = token[r];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = act_f32(embedding[size_t(tok) * width + c]) * scale;
    x[size_t(r) * width + c] = v;
    xa[size_t(r) * width + c] = to_act<T>(v);
  }
}

template <typename T>
struct QkvPostArgs {
  const float* qkv;   // [rows, H*d + G*d + G*dv]: the projection with its bias, or null:
  const bf16* qkv_bf16;  // the projection as the tcgen05 GEMM left it (bf16, no bias) and
  const float* bias;     // its bias [H*d + G*d + G*dv] (or null)
  const float* q_norm;  // [d] or null (no normalisation)
  const float* k_norm;  // [d] or null
  T* q_out;           // [rows, H*d]
  T* k_pages;         // [G, num_pages, tokens_per_page, d]
  T* v_pages;         // [G, num_pages, tokens_per_page, dv]
  float* v_shared;    // [rows, G*dv] values of the layer the others mix in (written when value_mix == 1, read when == 2)
  const int* group;
  const int* pos;
  const int* page_map;
  int heads, kv_heads, dim, vdim;
  int num_pages, tokens_per_page, max_pages;
  int value_mix;      // 0: none, 1: keep these values for later layers, 2: v = (1 - lambda) v + lambda v_shared
  float value_lambda, eps;
};

// one CTA per row; a warp per head for the norms
template <typename T>
__global__ void __launch_bounds__(256) qkv_post_kernel(const QkvPostArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim;
  const int n_all = H * d + G * d + G * dv;
  const float* rowf = a.qkv ? a.qkv + size_t(r) * n_all : nullptr;
  const bf16* rowb = a.qkv ? nullptr : a.qkv_bf16 + size_t(r) * n_all;
  auto val = [&](int c) { return rowf ? rowf[c] : __bfloat162float(rowb[c]) + (a.bias ? a.bias[c] : 0.0f); };
  const int p = a.pos[r], grp = a.group[r];
  const size_t slot = size_t(a.page_map[size_t(grp) * a.max_pages + p / a.tokens_per_page]) * a.tokens_per_page + p % a.tokens_per_page;
  for (int u = warp; u < H + G; u += nw) {  // unit u: query head u, or key head u - H
    const bool is_q = u < H;
    const int src = is_q ? u * d : H * d + (u - H) * d;
    const float* w = is_q ? a.q_norm : a.k_norm;
    float ss = 0.0f;
    for (int c = lane; c < d; c += 32) {
      const float v = val(src + c);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = w ? 1.0f / sqrtf(ss / float(d) + a.eps) : 1.0f;
    T* dst = is_q ? a.q_out + size_t(r) * H * d + u * d
                  : a.k_pages + (size_t(u - H) * a.num_pages * a.tokens_per_page + slot) * d;
    for (int c = lane; c < d; c += 32) dst[c] = to_act<T>(w ? val(src + c) * inv * w[c] : val(src + c));
  }
  const int vsrc = H * d + G * d;
  for (int e = tid; e < G * dv; e += blockDim.x) {
    float v = val(vsrc + e);
    if (a.value_mix == 1) a.v_shared[size_t(r) * G * dv + e] = v;
    else if (a.value_mix == 2) v = (1.0f - a.value_lambda) * v + a.value_lambda * a.v_shared[size_t(r) * G * dv + e];
    const int kv = e / dv, c = e % dv;
    a.v_pages[(size_t(kv) * a.num_pages * a.tokens_per_page + slot) * dv + c] = to_act<T>(v);
  }
}

// (y as fp32, or -- y null -- as the bf16 matrix y_bf16 a tcgen05 GEMM left)
template <typename T>
__global__ void __launch_bounds__(256) norm_residual_kernel(const float* y, const bf16* y_bf16, float gain, float eps, float* x, T* xa, int width) {
  __shared__ float red[8];
  griddep_wait();
  const int r = blockIdx.x;
  const float* yf = y ? y + size_t(r) * width : nullptr;
  const bf16* yb = y ? nullptr : y_bf16 + size_t(r) * width;
  auto val = [&](int c) { return yf ? yf[c] : __bfloat162float(yb[c]); };
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = val(c);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float f = gain / sqrtf(ss / float(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float v = x[size_t(r) * width + c] + val(c) * f;
    x[size_t(r) * width + c] = v;
    xa[size_t(r) * width + c] = to_act<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) scalar_norm_rows_kernel(const float* x, const int* rows, float gain, float eps, T* out, int width) {
  __shared__ float red[8];
  griddep_wait();
  const int src = rows ? rows[blockIdx.x] : int(blockIdx.x);
  const float* xr = x + size_t(src) * width;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
  ss = block_sum(ss, red);
  const float f = gain / sqrtf(ss / float(width) + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[size_t(blockIdx.x) * width + c] = to_act<T>(xr[c] * f);
}

}  // namespace mtx
