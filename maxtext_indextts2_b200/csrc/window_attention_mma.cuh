// Tensor-core arm of the windowed sigmoid attention (window_attention.cuh defines the operation and has the row kernel), bf16 operands.
//
// Work item = (query tile, key split).  A query tile is up to 16 rows of ONE sequence with consecutive positions (a slice of a
// prompt portion, or a single decoded token); the host passes the tile table.  Because the key weights are not normalised, the
// partial outputs of the key splits simply add: every work item writes its fp32 partial [rows, H * dv] and a small kernel sums the
// splits in a fixed order.  That is what lets 32 decode rows fill 148 SMs.
//
// One CTA of eight warps walks its keys in tiles of BN (32 or 64) staged in shared memory (K, V of all kv heads; rows fetched
// through the page map one by one, so any page size works).  Per tile:
//   S phase   warp w owns the keys [8w, 8w + 8) of the tile and ALL heads: S_g = Q_g K^T on mma.sync m16n8k16 (fp32 accumulators),
//             then scale, soft cap, distance bias, head bias, sigmoid and the window mask on the accumulator registers -- a thread
//             holds the same (row, key) element of every head, so the mixing of the heads' weights (an H x H matrix per element)
//             is thread-local.  The mixed weights go to shared memory as bf16 [H][16][BN].
//   PV phase  warp w owns HPW heads: out_h += P_h V_kv(h), V fragments through ldmatrix.trans.
// Template: HPW heads per warp (H <= 8 * HPW), DVT = ceil(dv / 8) output tiles per head; HPW * DVT * 4 accumulator registers.
#pragma once

#include "window_attention.cuh"

namespace mtx {

constexpr int kWmmaThreads = 256;
constexpr int kWmmaRows = 16;

struct WindowMmaExtra {
  const int* tile_row0;  // [n_tiles + 1]
  float* partial;        // [splits, rows, H * dv]
  int n_tiles, splits, bn;
  int hg;  // head groups of the S phase: 2 = two warps share a key group (bn = 32), each with half the heads; else 1
};

inline size_t window_mma_smem_bytes(int heads, int kv_heads, int dim, int vdim, int bn, int hg) {
  return size_t(2) * (size_t(kWmmaRows) * (heads * dim + 8) + size_t(kv_heads) * bn * (dim + 8) + size_t(kv_heads) * bn * (vdim + 8) +
                      size_t(heads) * kWmmaRows * (bn + 8)) +
         sizeof(float) * (size_t(heads) * 16 + heads + size_t(bn + kWmmaRows) * heads + (hg == 2 ? size_t(heads) * 4 * 4 * bn : 0)) +
         sizeof(int) * 64 + 16;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16 bytes global -> shared without a register round trip (all of a tile's rows are in flight at once); !valid: zeros
__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(n) : "memory");
}

// tanh to fp32 accuracy without the slow path of tanhf for the arguments a soft cap sees: |x| < 0.35 (a score of a third of
// the cap) takes the odd Taylor polynomial up to x^9 (error below 2e-8), anything larger 1 - 2 / (exp(2x) + 1).
__device__ __forceinline__ float tanh_f32(float x) {
  const float x2 = x * x;
  if (x2 < 0.1225f) return x * (1.0f + x2 * (-0.33333334f + x2 * (0.13333334f + x2 * (-0.05396825f + x2 * 0.02186949f))));
  return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f);
}

template <int HPW, int DVT>
__global__ void __launch_bounds__(kWmmaThreads, 1) window_attention_mma_kernel(const WindowAttnArgs<bf16> a, const WindowMmaExtra x) {
  constexpr int HMAX = 8 * HPW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim, BN = x.bn, rep = H / G;
  const int QP = H * d + 8, KP = d + 8, VP = dv + 8, PP = BN + 8;
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);      // [16][QP]
  bf16* sK = sQ + kWmmaRows * QP;                     // [G][BN][KP]
  bf16* sV = sK + G * BN * KP;                        // [G][BN][VP]
  bf16* sP = sV + G * BN * VP;                        // [H][16][PP]
  float* sTalk = reinterpret_cast<float*>(sP + H * kWmmaRows * PP);  // [H][HMAX]
  float* sPb = sTalk + H * HMAX;                      // [H]
  float* sBias = sPb + H;                             // [BN + 16][H] distance bias of the distances this tile can see
  int* sRow = reinterpret_cast<int*>(sBias + (BN + kWmmaRows) * H);  // [BN] cache row of each key of the tile (-1: none)
  float* sX = reinterpret_cast<float*>(sRow + 64);    // x.hg == 2: [H][4][4 * BN] raw weights, exchanged between the head groups
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g4 = lane >> 2, t4 = lane & 3;
  griddep_wait();
  const int tile = blockIdx.x, split = blockIdx.y;
  const int r0 = x.tile_row0[tile], nrows = x.tile_row0[tile + 1] - r0;
  const int grp = a.group[r0], p0 = a.pos[r0];
  const int klo = p0 - a.window + 1 > 0 ? p0 - a.window + 1 : 0, khi = p0 + nrows - 1;
  const int n_kt = (khi - klo + BN) / BN, per = (n_kt + x.splits - 1) / x.splits;
  const int kt_lo = split * per, kt_hi = (kt_lo + per < n_kt) ? kt_lo + per : n_kt;
  const int* pages = a.page_map + size_t(grp) * a.max_pages;

  // stage Q: only the tile's rows (the other rows of the MMA feed accumulator rows that are masked), the mixing matrix, the head bias
  {
    const int qch = H * d / 8;  // 16-byte chunks of a row
    for (int row = 0; row < nrows; ++row)
      for (int c8 = tid; c8 < qch; c8 += kWmmaThreads)
        *reinterpret_cast<uint4*>(sQ + row * QP + c8 * 8) = *reinterpret_cast<const uint4*>(a.q + size_t(r0 + row) * H * d + c8 * 8);
  }
  for (int e = tid; e < H * HMAX; e += kWmmaThreads) {
    const int h = e / HMAX, g = e % HMAX;
    sTalk[e] = g < H ? (a.talk ? a.talk[h * H + g] : (h == g ? 1.0f : 0.0f)) : 0.0f;
  }
  for (int e = tid; e < H; e += kWmmaThreads) sPb[e] = a.head_bias ? a.head_bias[e] : 0.0f;

  float acc[HPW][DVT][4];
#pragma unroll
  for (int u = 0; u < HPW; ++u)
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[u][nt][e] = 0.0f;

  const float inv_cap = a.softcap > 0.0f ? 1.0f / a.softcap : 0.0f;
  for (int kt = kt_lo; kt < kt_hi; ++kt) {
    const int j0 = klo + kt * BN;
    if (tid < BN) {
      const int j = j0 + tid;
      sRow[tid] = j <= khi ? pages[j / a.tokens_per_page] * a.tokens_per_page + j % a.tokens_per_page : -1;
    }
    __syncthreads();  // the previous tile's PV phase is over, the rows of this one are known
    {
      // the distances this tile's (row, key) pairs can have: p0 - (j0 + BN - 1) .. p0 + 15 - j0; slot n holds distance dist0 + n
      const int dist0 = p0 - j0 - BN + 1;
      for (int e = tid; e < (BN + kWmmaRows) * H; e += kWmmaThreads) {
        const int dd = dist0 + e / H;
        sBias[e] = (dd >= 0 && dd < a.window) ? __ldg(a.dist_bias + size_t(dd) * H + e % H) : 0.0f;
      }
      // K and V rows: thread t starts at (key, chunk) = (t / ch, t % ch) and walks 256 chunks further each time
      const int kch = d / 8, vch = dv / 8;
      const int kq = kWmmaThreads / kch, kr = kWmmaThreads % kch, vq = kWmmaThreads / vch, vr = kWmmaThreads % vch;
      for (int c = 0; c < G; ++c) {
        const bf16* kbase = a.k_pages + size_t(c) * a.num_pages * a.tokens_per_page * d;
        bf16* kdst = sK + c * BN * KP;
        for (int key = tid / kch, c8 = tid % kch; key < BN;) {
          const int row = sRow[key];
          cp_async_16(kdst + key * KP + c8 * 8, kbase + size_t(row < 0 ? 0 : row) * d + c8 * 8, row >= 0);
          key += kq;
          c8 += kr;
          if (c8 >= kch) {
            c8 -= kch;
            ++key;
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      for (int c = 0; c < G; ++c) {
        const bf16* vbase = a.v_pages + size_t(c) * a.num_pages * a.tokens_per_page * dv;
        bf16* vdst = sV + c * BN * VP;
        for (int key = tid / vch, c8 = tid % vch; key < BN;) {
          const int row = sRow[key];
          cp_async_16(vdst + key * VP + c8 * 8, vbase + size_t(row < 0 ? 0 : row) * dv + c8 * 8, row >= 0);
          key += vq;
          c8 += vr;
          if (c8 >= vch) {
            c8 -= vch;
            ++key;
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // K has landed; V keeps flying under the S phase
    __syncthreads();
    // ---- S phase: this warp's 8 keys; every head, or (two head groups) its half of the heads ----
    const int KG = BN >> 3, kg = warp % KG, hg = warp / KG;  // key group, head group
    const int hpg = H / x.hg, h_lo = hg * hpg, h_hi = h_lo + hpg;
    if (hg < x.hg) {
      float w[HMAX][4];
      // the four weights of head g that this thread's accumulator elements hold: (rows g4, g4 + 8) x (keys 2 t4, 2 t4 + 1)
      auto head_weights = [&](int g, float (&out)[4]) {
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const bf16* qb = sQ + g4 * QP + g * d + 2 * t4;
        const bf16* kb = sK + ((g / rep) * BN + kg * 8 + g4) * KP + 2 * t4;
        for (int ks = 0; ks < d; ks += 16) {
          uint32_t af[4];
          af[0] = *reinterpret_cast<const uint32_t*>(qb + ks);
          af[1] = *reinterpret_cast<const uint32_t*>(qb + ks + 8 * QP);
          af[2] = *reinterpret_cast<const uint32_t*>(qb + ks + 8);
          af[3] = *reinterpret_cast<const uint32_t*>(qb + ks + 8 * QP + 8);
          mma_bf16_16816(s, af, *reinterpret_cast<const uint32_t*>(kb + ks), *reinterpret_cast<const uint32_t*>(kb + ks + 8));
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ir = g4 + (e >> 1) * 8, jj = kg * 8 + 2 * t4 + (e & 1), dist = p0 + ir - j0 - jj;
          float wv = 0.0f;
          if (ir < nrows && dist >= 0 && dist < a.window) {
            float sc = s[e] * a.scale;
            if (a.softcap > 0.0f) sc = a.softcap * tanh_f32(sc * inv_cap);
            sc += sBias[(ir + BN - 1 - jj) * H + g] + sPb[g];
            wv = __fdividef(1.0f, 1.0f + __expf(-sc));
          }
          out[e] = wv;
        }
      };
      if (x.hg == 2) {
        // two warps share a key group: each computes the weights of half the heads, they meet in shared memory ([head][element]
        // [thread of the key group]: conflict-free), and each mixes for its own half of the output heads
        float* xw = sX + kg * 32 + lane;
#pragma unroll
        for (int gl = 0; gl < HMAX / 2; ++gl) {
          if (gl < hpg) {
            float o[4];
            head_weights(h_lo + gl, o);
#pragma unroll
            for (int e = 0; e < 4; ++e) xw[((h_lo + gl) * 4 + e) * (KG * 32)] = o[e];
          }
        }
        __syncthreads();  // (every warp is here: x.hg == 2 means KG * 2 == 8 warps)
#pragma unroll
        for (int g = 0; g < HMAX; ++g) {
          if (g < H) {
#pragma unroll
            for (int e = 0; e < 4; ++e) w[g][e] = xw[(g * 4 + e) * (KG * 32)];
          }
        }
      } else {
#pragma unroll
        for (int g = 0; g < HMAX; ++g) {
          if (g < H) head_weights(g, w[g]);
        }
      }
      // mix the heads' weights; P_h as bf16
#pragma unroll 1
      for (int h = h_lo; h < h_hi; ++h) {
        float m[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* tr = sTalk + h * HMAX;  // (rows padded to HMAX floats: 16-byte reads, zeros beyond H)
#pragma unroll
        for (int g = 0; g < HMAX; g += 4) {
          if (g < H) {
            const float4 tv = *reinterpret_cast<const float4*>(tr + g);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              m[e] = fmaf(tv.x, w[g][e], m[e]);
              if (g + 1 < H) m[e] = fmaf(tv.y, w[g + 1][e], m[e]);
              if (g + 2 < H) m[e] = fmaf(tv.z, w[g + 2][e], m[e]);
              if (g + 3 < H) m[e] = fmaf(tv.w, w[g + 3][e], m[e]);
            }
          }
        }
        bf16* pb = sP + (h * kWmmaRows + g4) * PP + kg * 8 + 2 * t4;
        *reinterpret_cast<uint32_t*>(pb) = pack_bf16x2(m[0], m[1]);
        *reinterpret_cast<uint32_t*>(pb + 8 * PP) = pack_bf16x2(m[2], m[3]);
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's part of V
    __syncthreads();
    // ---- PV phase: this warp's heads ----
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
      const int h = warp * HPW + u;
      if (h < H) {
        const bf16* pb = sP + (h * kWmmaRows + g4) * PP + 2 * t4;
        const bf16* vb = sV + (h / rep) * BN * VP;
        for (int k2 = 0; k2 < BN; k2 += 16) {
          uint32_t af[4];
          af[0] = *reinterpret_cast<const uint32_t*>(pb + k2);
          af[1] = *reinterpret_cast<const uint32_t*>(pb + k2 + 8 * PP);
          af[2] = *reinterpret_cast<const uint32_t*>(pb + k2 + 8);
          af[3] = *reinterpret_cast<const uint32_t*>(pb + k2 + 8 * PP + 8);
#pragma unroll
          for (int nt = 0; nt < DVT; ++nt) {
            if (nt * 8 < dv) {
              uint32_t b0, b1;
              const uint32_t addr = smem_u32(vb + (k2 + (lane & 15)) * VP + nt * 8);  // lanes 0-15: the 16 key rows of this k step
              asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
              mma_bf16_16816(acc[u][nt], af, b0, b1);
            }
          }
        }
      }
    }
  }
  // this split's partial sums (zeros if it had no keys)
  const size_t out_row = size_t(H) * dv;
  float* part = x.partial + size_t(split) * a.rows * out_row;
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    const int h = warp * HPW + u;
    if (h < H) {
#pragma unroll
      for (int nt = 0; nt < DVT; ++nt) {
        if (nt * 8 < dv) {
          const int col = h * dv + nt * 8 + 2 * t4;
          if (g4 < nrows) *reinterpret_cast<float2*>(part + size_t(r0 + g4) * out_row + col) = make_float2(acc[u][nt][0], acc[u][nt][1]);
          if (g4 + 8 < nrows) *reinterpret_cast<float2*>(part + size_t(r0 + g4 + 8) * out_row + col) = make_float2(acc[u][nt][2], acc[u][nt][3]);
        }
      }
    }
  }
}

// out[r, o] = bf16(sum over the splits, in order)
__global__ void window_partial_sum_kernel(const float* partial, bf16* out, int splits, long long per_split) {
  griddep_wait();
  for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 2; i < per_split; i += (long long)gridDim.x * blockDim.x * 2) {
    float2 s = *reinterpret_cast<const float2*>(partial + i);
    for (int p = 1; p < splits; ++p) {
      const float2 v = *reinterpret_cast<const float2*>(partial + p * per_split + i);
      s.x += v.x;
      s.y += v.y;
    }
    *reinterpret_cast<uint32_t*>(out + i) = pack_bf16x2(s.x, s.y);
  }
}

struct WindowMmaPlan {
  bool ok = false;
  int hpw = 0, dvt = 0, bn = 0, hg = 1;
  size_t smem = 0;
};

// Which instantiation serves this head geometry, if any: bf16, dim and vdim multiples of 16 (fragments and 16-byte rows), at most
// 16 heads, HPW * DVT <= 32 accumulator tiles per thread, shared memory within the SM's.
inline WindowMmaPlan window_mma_plan(int heads, int kv_heads, int dim, int vdim) {
  WindowMmaPlan p;
  if (dim % 16 != 0 || vdim % 16 != 0 || heads > 16 || heads % kv_heads != 0) return p;
  p.hpw = heads <= 8 ? 1 : 2;
  const int need = (vdim + 7) / 8;
  p.dvt = need <= 8 ? 8 : (need <= 16 ? 16 : 32);
  if (need > 32 || p.hpw * p.dvt > 32) return p;
  // 64-key tiles (every warp a key group of its own) if they fit; else 32-key tiles with the heads split over two warps per key
  // group (an even head count, and room for the exchange buffer); else 32-key tiles with half the warps idle in the S phase
  const int tries[3][2] = {{64, 1}, {32, 2}, {32, 1}};
  for (const auto& t : tries) {
    if (t[1] == 2 && heads % 2 != 0) continue;
    const size_t s = window_mma_smem_bytes(heads, kv_heads, dim, vdim, t[0], t[1]);
    if (s <= 227 * 1024) {  // the most a CTA can have
      p.bn = t[0];
      p.hg = t[1];
      p.smem = s;
      p.ok = true;
      return p;
    }
  }
  return p;
}

}  // namespace mtx
