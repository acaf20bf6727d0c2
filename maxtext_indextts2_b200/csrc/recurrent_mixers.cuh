// Linear recurrences with a matrix state per head, over a ragged batch and a pool of state slots.
//
// Per head, with q, k of size d, v of size dv and the state S [d, dv] (fp32, one per page group and layer run):
//
//   GLA    S <- diag(a) S + k v^T,  o = S^T q                      a = sigmoid(z)^(1 / tau) per key channel
//   mLSTM  m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone;
//          o = S^T q / (max(|n . q|, e^(-m')) + denom_eps)          (m starts at 0; i, f are log gates)
//
// A run (consecutive rows of one sequence) is walked in order from the group's state; a run that starts at position 0 starts
// from zero instead, so a slot that is handed to another sequence needs no clearing.  Every value column of S is independent of
// the others, so a (run, head) is spread over CTAs by column block: a CTA keeps its columns of S in registers (8 row slices x
// 16 columns), stages the run's q / k / decays / v in chunks through shared memory and walks the tokens one by one.  The result
// of a token is the same bits however the sequence is cut into steps.
//
//   recurrent_prepare_kernel   per row: the GLA's decays (low-rank up-projection, bias, sigmoid^(1/tau)) or the mLSTM's two log gates
//   recurrent_scan_kernel      the walk
//   recurrent_out_kernel<T>    per row and head: o / rms(o) * weight * gate(g) * out_scale -> the activation of the output projection
#pragma once

#include "common.cuh"
#include "layer_ops.cuh"
#include "linear_any.cuh"

namespace mtx {

enum { REC_GLA = 1, REC_MLSTM = 2 };

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

struct RecPrepareArgs {
  const float* proj;  // [rows, ld]
  long long ld;
  int x_col;          // GLA: first of the decay_rank down-projection columns; mLSTM: first input-gate column (forget gates follow)
  int kind, heads, dim, rank;
  float tau, cap;
  const float* up_t;  // GLA [rank, heads * dim]
  const float* bias;  // GLA [heads * dim]; mLSTM [2 * heads]
  float* out;         // GLA [rows, heads * dim] decays; mLSTM [rows, 2 * heads] log gates (input, then forget)
};

__global__ void __launch_bounds__(256) recurrent_prepare_kernel(const RecPrepareArgs a) {
  extern __shared__ float s_low[];
  griddep_wait();
  const int r = blockIdx.x;
  const float* row = a.proj + size_t(r) * a.ld + a.x_col;
  if (a.kind == REC_GLA) {
    const int n = a.heads * a.dim;
    for (int e = threadIdx.x; e < a.rank; e += blockDim.x) s_low[e] = row[e];
    __syncthreads();
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float z = a.bias ? a.bias[c] : 0.0f;
      for (int e = 0; e < a.rank; ++e) z = fmaf(a.up_t[size_t(e) * n + c], s_low[e], z);
      a.out[size_t(r) * n + c] = expf(log_sigmoid_f(z) / a.tau);
    }
  } else {
    const int H = a.heads;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float ig = a.cap * tanhf((row[h] + a.bias[h]) / a.cap);
      const float fg = log_sigmoid_f(a.cap * tanhf((row[H + h] + a.bias[H + h]) / a.cap));
      a.out[size_t(r) * 2 * H + h] = ig;
      a.out[size_t(r) * 2 * H + H + h] = fg;
    }
  }
}

struct RecScanArgs {
  const float* proj;   // [rows, ld]: q at q_col, k at k_col, v at v_col (heads x dim, heads x dim, heads x vdim)
  long long ld;
  int q_col, k_col, v_col;
  const float* aux;    // the prepare kernel's output
  float* o;            // [rows, heads * vdim]
  float* state_s;      // [slots, heads, dim, vdim]
  float* state_n;      // mLSTM [slots, heads, dim]
  float* state_m;      // mLSTM [slots, heads]
  const int* run_row0; // [n_runs + 1]
  const int* group;
  const int* pos;
  int heads, dim, vdim, chunk;
  float q_scale, denom_eps;
};

constexpr int kRecThreads = 128, kRecCols = 16, kRecSlices = 8;

inline int rec_chunk_tokens(int dim) {
  int t = (40 * 1024) / int(sizeof(float) * (3 * dim + kRecCols + 2));
  return t > 16 ? 16 : (t < 1 ? 1 : t);
}
inline size_t rec_scan_smem_bytes(int dim, int chunk) { return sizeof(float) * size_t(chunk) * (3 * dim + kRecCols + 2); }

template <int KIND, int RPT>
__global__ void __launch_bounds__(kRecThreads) recurrent_scan_kernel(const RecScanArgs a) {
  extern __shared__ float smem[];
  const int d = a.dim, dv = a.vdim, H = a.heads, TC = a.chunk;
  float* sq = smem;            // [TC][d]
  float* sk = sq + TC * d;     // [TC][d]
  float* sa = sk + TC * d;     // [TC][d] decays (GLA)
  float* sv = sa + TC * d;     // [TC][16]
  float* sg = sv + TC * kRecCols;  // [TC][2] log gates (mLSTM)
  const int tid = threadIdx.x, jl = tid >> 3, sl = tid & 7;
  griddep_wait();
  const int r0 = a.run_row0[blockIdx.x], nr = a.run_row0[blockIdx.x + 1] - r0, h = blockIdx.y;
  if (nr <= 0) return;
  const int col0 = blockIdx.z * kRecCols, j = col0 + jl;
  const bool col_ok = j < dv;
  const int slot = a.group[r0];
  const bool fresh = a.pos[r0] == 0;
  float S[RPT], N[RPT];
  float m = 0.0f;
  float* gs = a.state_s + (size_t(slot) * H + h) * d * dv;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = sl + kRecSlices * i;
    S[i] = (!fresh && col_ok && r < d) ? gs[size_t(r) * dv + j] : 0.0f;
    N[i] = 0.0f;
  }
  if (KIND == REC_MLSTM && !fresh) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = sl + kRecSlices * i;
      if (r < d) N[i] = a.state_n[(size_t(slot) * H + h) * d + r];
    }
    m = a.state_m[size_t(slot) * H + h];
  }
  for (int t0 = 0; t0 < nr; t0 += TC) {
    const int nt = nr - t0 < TC ? nr - t0 : TC;
    __syncthreads();
    for (int e = tid; e < nt * d; e += kRecThreads) {
      const int t = e / d, c = e % d;
      const float* row = a.proj + size_t(r0 + t0 + t) * a.ld;
      sq[e] = row[a.q_col + h * d + c] * a.q_scale;
      sk[e] = row[a.k_col + h * d + c];
      if (KIND == REC_GLA) sa[e] = a.aux[size_t(r0 + t0 + t) * H * d + h * d + c];
    }
    for (int e = tid; e < nt * kRecCols; e += kRecThreads) {
      const int t = e / kRecCols, c = e % kRecCols;
      sv[e] = col0 + c < dv ? a.proj[size_t(r0 + t0 + t) * a.ld + a.v_col + h * dv + col0 + c] : 0.0f;
    }
    if (KIND == REC_MLSTM) {
      for (int e = tid; e < nt * 2; e += kRecThreads) {
        const int t = e >> 1, w = e & 1;
        sg[e] = a.aux[size_t(r0 + t0 + t) * 2 * H + w * H + h];
      }
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float* q = sq + t * d;
      const float* k = sk + t * d;
      const float v = sv[t * kRecCols + jl];
      float part = 0.0f, npart = 0.0f, floor_m = 0.0f;
      if (KIND == REC_GLA) {
        const float* al = sa + t * d;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int r = sl + kRecSlices * i;
          if (r < d) {
            S[i] = fmaf(al[r], S[i], k[r] * v);
            part = fmaf(S[i], q[r], part);
          }
        }
      } else {
        const float ig = sg[2 * t], fg = sg[2 * t + 1];
        const float m_new = fmaxf(fg + m, ig);
        const float keep = expf(fg + m - m_new), put = expf(ig - m_new);
        m = m_new;
        floor_m = expf(-m_new);
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int r = sl + kRecSlices * i;
          if (r < d) {
            const float pk = put * k[r];
            S[i] = fmaf(keep, S[i], pk * v);
            N[i] = fmaf(keep, N[i], pk);
            part = fmaf(S[i], q[r], part);
            npart = fmaf(N[i], q[r], npart);
          }
        }
      }
#pragma unroll
      for (int o = 1; o < kRecSlices; o <<= 1) {
        part += __shfl_xor_sync(0xffffffffu, part, o);
        if (KIND == REC_MLSTM) npart += __shfl_xor_sync(0xffffffffu, npart, o);
      }
      if (sl == 0 && col_ok) {
        float out = part;
        if (KIND == REC_MLSTM) out = part / (fmaxf(fabsf(npart), floor_m) + a.denom_eps);
        a.o[size_t(r0 + t0 + t) * H * dv + h * dv + j] = out;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = sl + kRecSlices * i;
    if (col_ok && r < d) gs[size_t(r) * dv + j] = S[i];
  }
  if (KIND == REC_MLSTM && blockIdx.z == 0 && jl == 0) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int r = sl + kRecSlices * i;
      if (r < d) a.state_n[(size_t(slot) * H + h) * d + r] = N[i];
    }
    if (sl == 0) a.state_m[size_t(slot) * H + h] = m;
  }
}

template <typename T>
struct RecOutArgs {
  const float* o;       // [rows, heads * vdim]
  const float* proj;    // [rows, ld]: the output gate's pre-activation at g_col
  long long ld;
  int g_col;
  const float* weight;  // [heads * vdim]
  T* out;               // [rows, ld_out], written from column out_col
  long long ld_out;
  int out_col;
  int heads, vdim, gate_silu;
  float eps, out_scale;
};

// one CTA per row, a warp per head
template <typename T>
__global__ void __launch_bounds__(256) recurrent_out_kernel(const RecOutArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, dv = a.vdim;
  for (int h = warp; h < a.heads; h += nw) {
    const float* o = a.o + size_t(r) * a.heads * dv + h * dv;
    float ss = 0.0f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / float(dv) + a.eps);
    for (int c = lane; c < dv; c += 32) {
      const float g = a.proj[size_t(r) * a.ld + a.g_col + h * dv + c];
      const float sig = 1.0f / (1.0f + expf(-g));
      const float gate = a.gate_silu ? g * sig : sig;
      a.out[size_t(r) * a.ld_out + a.out_col + h * dv + c] = to_act<T>(o[c] * inv * a.weight[h * dv + c] * gate * a.out_scale);
    }
  }
}

}  // namespace mtx
