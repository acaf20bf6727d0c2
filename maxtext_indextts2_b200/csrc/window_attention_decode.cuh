// Decode arm of the windowed sigmoid attention (window_attention.cuh defines the operation): every row of the step is a single token
// of its own sequence, so the kernel is bound by reading each row's window of K and V once.  bf16 operands.
//
// Work item = (row, key split); the key weights are not normalised, so the splits' fp32 partial outputs add (summed in a fixed
// order by window_partial_sum_kernel).  One CTA of four warps walks its keys in tiles of 16, K and V of all kv heads staged by
// cp.async in a ring of `stages` buffers (stages - 1 tiles in flight while one is computed; CTAs are small enough that several
// share an SM).  With one query row the 16-row MMA of the prefill arm would be 15/16 idle, so the roles are swapped here: the
// KEYS are the M dimension and the (up to 8) query heads of a kv head the N dimension.
//   S phase   warp w, kv head c = w, w + 4, ..: S^T[16 keys, 8 heads] = K_c Q_c^T on mma.sync m16n8k16 (K through ldmatrix), then
//             scale, soft cap, distance bias, head bias, sigmoid and the window mask in fp32 -> sW[key][head] (fp32)
//   mix       all threads: P_h(key) = sum_g talk[h, g] * W_g(key) in fp32 -> sP[head slot][key] (bf16)
//   PV phase  warp w, kv head c: out^T[dv, 8 heads] += V_c^T P^T, V through ldmatrix.trans
// Template: CPW kv heads per warp (G <= 4 * CPW), DT = ceil(dv / 16) value tiles; CPW * DT * 4 accumulator registers.
#pragma once

#include "window_attention_mma.cuh"

namespace mtx {

constexpr int kWdecThreads = 128;
constexpr int kWdecKeys = 16;

struct WindowDecodeExtra {
  float* partial;  // [splits, rows, H * dv]
  int splits, stages;
};

inline size_t window_decode_tile_bytes(int kv_heads, int dim, int vdim) {
  return size_t(2) * kv_heads * kWdecKeys * (size_t(dim + 8) + size_t(vdim + 8));
}

inline size_t window_decode_smem_bytes(int heads, int kv_heads, int dim, int vdim, int stages) {
  return size_t(2) * (size_t(kv_heads) * 8 * (dim + 8) + size_t(kv_heads) * 8 * (kWdecKeys + 8)) +
         size_t(stages) * window_decode_tile_bytes(kv_heads, dim, vdim) +
         sizeof(float) * (size_t(kWdecKeys) * (heads + 1) + size_t(heads) * heads + 2 * size_t(heads)) + 16;
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// wait until at most n of this thread's committed groups are pending (n = 0..2)
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  if (n <= 0) asm volatile("cp.async.wait_group 0;" ::: "memory");
  else if (n == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else asm volatile("cp.async.wait_group 2;" ::: "memory");
}

template <int CPW, int DT>
__global__ void __launch_bounds__(kWdecThreads) window_attention_decode_kernel(const WindowAttnArgs<bf16> a, const WindowDecodeExtra x) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim, rep = H / G, NS = x.stages;
  const int QP = d + 8, VP = dv + 8, PP = kWdecKeys + 8, WP = H + 1;
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);         // [G * 8][QP]: head hh of kv head c in row c * 8 + hh, zeros beyond rep
  bf16* sP = sQ + G * 8 * QP;                            // [G * 8][PP] mixed weights of the tile
  bf16* sK = sP + G * 8 * PP;                            // [NS][G][16][QP]
  bf16* sV = sK + size_t(NS) * G * kWdecKeys * QP;       // [NS][G][16][VP]
  float* sW = reinterpret_cast<float*>(sV + size_t(NS) * G * kWdecKeys * VP);  // [16][WP] raw weights of the tile
  float* sTalk = sW + kWdecKeys * WP;                    // [H][H]
  float* sPb = sTalk + H * H;                            // [H]
  int* sSlot = reinterpret_cast<int*>(sPb + H);          // [H] row of sP that holds head h: (h / rep) * 8 + h % rep
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g4 = lane >> 2, t4 = lane & 3;
  griddep_wait();
  const int r = blockIdx.x, split = blockIdx.y;
  const int i = a.pos[r], grp = a.group[r];
  const int klo = i - a.window + 1 > 0 ? i - a.window + 1 : 0;
  const int n_kt = (i - klo + kWdecKeys) / kWdecKeys, per = (n_kt + x.splits - 1) / x.splits;
  const int kt_lo = split * per, kt_hi = (kt_lo + per < n_kt) ? kt_lo + per : n_kt;
  const int n = kt_hi > kt_lo ? kt_hi - kt_lo : 0;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;
  const size_t kv_rows = size_t(a.num_pages) * a.tokens_per_page;
  const int tpp_shift = (a.tokens_per_page & (a.tokens_per_page - 1)) == 0 ? __ffs(a.tokens_per_page) - 1 : -1;

  // tile t of this split -> ring slot t % NS: thread (key = tid / 8, lane-of-key = tid % 8) copies every 8th 16-byte chunk of
  // its key's K and V rows of every kv head; keys beyond the row's own position are zero-filled (and masked below)
  auto issue = [&](int t) {
    const int st = t % NS, kk = tid >> 3, sub = tid & 7;
    const int j = klo + (kt_lo + t) * kWdecKeys + kk;
    const bool valid = j <= i;
    const int pg = tpp_shift >= 0 ? j >> tpp_shift : j / a.tokens_per_page, in_pg = j - pg * a.tokens_per_page;
    const size_t row = valid ? size_t(pages[pg]) * a.tokens_per_page + in_pg : 0;
    const int kch = d >> 3, vch = dv >> 3;
    const bf16* ksrc = a.k_pages + row * d + sub * 8;
    const bf16* vsrc = a.v_pages + row * dv + sub * 8;
    uint32_t kdst = smem_u32(sK + (size_t(st) * G * kWdecKeys + kk) * QP + sub * 8);
    uint32_t vdst = smem_u32(sV + (size_t(st) * G * kWdecKeys + kk) * VP + sub * 8);
    const int nbytes = valid ? 16 : 0;
    for (int c = 0; c < G; ++c) {
      for (int c8 = sub; c8 < kch; c8 += 8)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kdst + (c8 - sub) * 16), "l"(ksrc + (c8 - sub) * 8), "r"(nbytes) : "memory");
      for (int c8 = sub; c8 < vch; c8 += 8)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vdst + (c8 - sub) * 16), "l"(vsrc + (c8 - sub) * 8), "r"(nbytes) : "memory");
      ksrc += kv_rows * d;
      vsrc += kv_rows * dv;
      kdst += kWdecKeys * QP * 2;
      vdst += kWdecKeys * VP * 2;
    }
  };
  for (int s = 0; s < NS - 1; ++s) {
    if (s < n) issue(s);
    cp_async_commit();
  }
  // the row's queries, the mixing matrix, the head bias (visible after the loop's first barrier)
  for (int e = tid; e < G * 8 * (d >> 3); e += kWdecThreads) {
    const int slot = e / (d >> 3), c8 = e % (d >> 3), c = slot >> 3, hh = slot & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (hh < rep) v = *reinterpret_cast<const uint4*>(a.q + (size_t(r) * H + c * rep + hh) * d + c8 * 8);
    *reinterpret_cast<uint4*>(sQ + slot * QP + c8 * 8) = v;
  }
  for (int e = tid; e < H * H; e += kWdecThreads) sTalk[e] = a.talk ? a.talk[e] : ((e / H == e % H) ? 1.0f : 0.0f);
  for (int e = tid; e < H; e += kWdecThreads) {
    sPb[e] = a.head_bias ? a.head_bias[e] : 0.0f;
    sSlot[e] = (e / rep) * 8 + e % rep;
  }
  for (int e = tid; e < G * 8 * PP; e += kWdecThreads) sP[e] = __float2bfloat16(0.0f);  // slots beyond rep stay zero

  float acc[CPW][DT][4];
#pragma unroll
  for (int u = 0; u < CPW; ++u)
#pragma unroll
    for (int mt = 0; mt < DT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[u][mt][e] = 0.0f;

  const float inv_cap = a.softcap > 0.0f ? 1.0f / a.softcap : 0.0f;
  for (int t = 0; t < n; ++t) {
    cp_async_wait_pending(NS - 2);  // tile t has landed (this thread's part)
    __syncthreads();                // ... everyone's; and the previous tile's PV phase is over, so its slot may be refilled
    if (t + NS - 1 < n) issue(t + NS - 1);
    cp_async_commit();
    const int st = t % NS, j0 = klo + (kt_lo + t) * kWdecKeys;
    // ---- S phase ----
#pragma unroll
    for (int u = 0; u < CPW; ++u) {
      const int c = warp + 4 * u;
      if (c < G) {
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // this thread's four (key, head) elements: their distance biases are fetched before the MMA chain, which hides the loads
        float db[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int hh = 2 * t4 + (e & 1), dist = i - (j0 + g4 + (e >> 1) * 8);
          db[e] = (hh < rep && dist >= 0 && dist < a.window) ? __ldg(a.dist_bias + size_t(dist) * H + c * rep + hh) : 0.0f;
        }
        const bf16* kb = sK + ((size_t(st) * G + c) * kWdecKeys + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + (lane >> 4) * 8;
        const bf16* qb = sQ + (c * 8 + g4) * QP + 2 * t4;
#pragma unroll 4
        for (int ks = 0; ks < d; ks += 16) {
          uint32_t af[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3])
                       : "r"(smem_u32(kb + ks)));
          mma_bf16_16816(s, af, *reinterpret_cast<const uint32_t*>(qb + ks), *reinterpret_cast<const uint32_t*>(qb + ks + 8));
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kk = g4 + (e >> 1) * 8, hh = 2 * t4 + (e & 1), dist = i - (j0 + kk);
          if (hh < rep) {
            const int g = c * rep + hh;
            float wv = 0.0f;
            if (dist >= 0 && dist < a.window) {
              float sc = s[e] * a.scale;
              if (a.softcap > 0.0f) sc = a.softcap * tanh_f32(sc * inv_cap);
              sc += db[e] + sPb[g];
              wv = __fdividef(1.0f, 1.0f + __expf(-sc));
            }
            sW[kk * WP + g] = wv;
          }
        }
      }
    }
    __syncthreads();
    // ---- mix the heads' weights ----
    {
      const int kk = tid & (kWdecKeys - 1);  // (128 threads = 8 heads x 16 keys per pass)
      const float* wr = sW + kk * WP;
      for (int h = tid >> 4; h < H; h += kWdecThreads / kWdecKeys) {
        const float* tr = sTalk + h * H;
        float m = 0.0f;
#pragma unroll 4
        for (int g = 0; g < H; ++g) m = fmaf(tr[g], wr[g], m);
        sP[sSlot[h] * PP + kk] = __float2bfloat16(m);
      }
    }
    __syncthreads();
    // ---- PV phase ----
#pragma unroll
    for (int u = 0; u < CPW; ++u) {
      const int c = warp + 4 * u;
      if (c < G) {
        const bf16* pb = sP + (c * 8 + g4) * PP + 2 * t4;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(pb), b1 = *reinterpret_cast<const uint32_t*>(pb + 8);
        const bf16* vb = sV + ((size_t(st) * G + c) * kWdecKeys + (lane & 7) + (lane >> 4) * 8) * VP + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int mt = 0; mt < DT; ++mt) {
          if (mt * 16 < dv) {
            uint32_t af[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(af[0]), "=r"(af[1]), "=r"(af[2]), "=r"(af[3])
                         : "r"(smem_u32(vb + mt * 16)));
            mma_bf16_16816(acc[u][mt], af, b0, b1);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // this split's partial sums (zeros if it had no keys): accumulator element = (value column, head)
  float* part = x.partial + (size_t(split) * a.rows + r) * H * dv;
#pragma unroll
  for (int u = 0; u < CPW; ++u) {
    const int c = warp + 4 * u;
    if (c < G) {
#pragma unroll
      for (int mt = 0; mt < DT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = mt * 16 + g4 + (e >> 1) * 8, hh = 2 * t4 + (e & 1);
          if (col < dv && hh < rep) part[size_t(c * rep + hh) * dv + col] = acc[u][mt][e];
        }
      }
    }
  }
}

struct WindowDecodePlan {
  bool ok = false;
  int cpw = 0, dt = 0, stages = 0;
  size_t smem = 0;
};

// Which instantiation serves this head geometry, if any: dim and vdim multiples of 16, at most 8 query heads per kv head, at most
// 8 kv heads, CPW * DT <= 16 accumulator tiles.  The ring is as shallow as it can be (two buffers, or `force_stages`): the kernel is
// bound by the instructions it issues per tile, not by bytes in flight, so the CTAs that a smaller ring lets share an SM are worth
// more than a deeper ring (measured: two buffers beat three and four clearly at two of three geometries and lose 4 % at the third).
inline WindowDecodePlan window_decode_plan(int heads, int kv_heads, int dim, int vdim, int force_stages) {
  WindowDecodePlan p;
  if (dim % 16 != 0 || vdim % 16 != 0 || kv_heads < 1 || heads % kv_heads != 0 || heads / kv_heads > 8 || kv_heads > 8 || heads > 64) return p;
  p.cpw = kv_heads <= 4 ? 1 : 2;
  const int need = vdim / 16;
  p.dt = need <= 4 ? 4 : (need <= 8 ? 8 : 16);
  if (need > 16 || p.cpw * p.dt > 16) return p;
  for (int ns = 2; ns <= 4; ++ns) {
    if (force_stages >= 2 && ns != force_stages) continue;
    const size_t s = window_decode_smem_bytes(heads, kv_heads, dim, vdim, ns);
    if (s > 220 * 1024) continue;
    p.stages = ns;
    p.smem = s;
    p.ok = true;
    break;
  }
  return p;
}

}  // namespace mtx
