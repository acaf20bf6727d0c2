// The layered engine of include/mtx_b200.h (mtx_layered_*): a decoder given as a list of layer descriptors, stepped over ragged
// batches whose keys and values live in page pools.  Host code only: the kernels are in linear_any.cuh (any-shape projections),
// gemm_rows.cuh (the tcgen05 projections, for shapes made of whole 128 x 64 tiles), layer_ops.cuh (norms, residual, cache
// append) and window_attention.cuh / window_attention_mma.cuh (the mixer).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../include/mtx_b200.h"
#include "layer_ops.cuh"
#include "linear_any.cuh"
#include "window_attention.cuh"
#include "window_attention_mma.cuh"
#include "window_attention_decode.cuh"
#include "host_util.cuh"

using namespace mtx;

struct mtx_layered {
  mtx_layered_config cfg;
  std::vector<mtx_layer_desc> layers;
  int num_sms = 148;
  int max_nqkv = 0, max_qdim = 0, max_odim = 0, max_ff = 0, vshared_dim = 0;
  size_t ws_bytes = 0;
  bool bound = false;
  // workspace carve-up
  float *x = nullptr, *y = nullptr, *qkv = nullptr, *v_shared = nullptr;
  void *xa = nullptr, *q = nullptr, *attn = nullptr, *act = nullptr, *wanted = nullptr, *obf = nullptr;
  // mtx_layered_step_graph: one instantiated graph per distinct batch descriptor (a decode loop passes the same one every step)
  struct GraphEntry {
    mtx_ragged_batch key;
    cudaGraphExec_t exec;
  };
  std::vector<GraphEntry> graphs;
  cudaStream_t cap_stream = nullptr;
  float* attn_part = nullptr;  // fp32 partial outputs of the attention's key splits: room for 4 * max_rows rows
  size_t attn_part_rows = 0;
};

namespace {

size_t elem(const mtx_layered* e) { return e->cfg.float32 ? 4 : 2; }

struct LWs {
  size_t x, y, qkv, v_shared, xa, q, attn, act, wanted, obf, attn_part, total;
};

LWs layered_layout(const mtx_layered* e) {
  const mtx_layered_config& c = e->cfg;
  // (rows padded to a multiple of 256: the tcgen05 projections read whole row blocks)
  const size_t R = align_up(size_t(c.max_rows), 256), W = align_up(size_t(c.max_want > 0 ? c.max_want : 1), 256), es = elem(e);
  LWs L;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes, 1024);
    return at;
  };
  L.x = take(R * c.width * 4);
  L.y = take(R * c.width * 4);
  L.qkv = take(R * e->max_nqkv * 4);
  L.v_shared = take(R * (e->vshared_dim > 0 ? e->vshared_dim : 1) * 4);
  L.xa = take(R * c.width * es);
  L.q = take(R * e->max_qdim * es);
  L.attn = take(R * e->max_odim * es);
  L.act = take(R * (e->max_ff > 0 ? e->max_ff : 1) * es);
  L.wanted = take(W * c.width * es);
  L.obf = take(R * size_t(e->max_nqkv > c.width ? e->max_nqkv : c.width) * 2);  // bf16 output of a tcgen05 projection
  L.attn_part = take(c.float32 ? 1024 : 4 * R * size_t(e->max_odim) * 4);
  L.total = off;
  return L;
}

// does the projection [rows, k] x [n, k] fit the tcgen05 GEMM of gemm_rows.cuh?  (whole 128-column weight tiles, 64-element k blocks,
// 16-byte aligned rows for TMA)
bool fits_umma(const mtx_layered* e, int n, int k) {
  static int on = env_int("MTX_LAYERED_UMMA", 1);
  return on != 0 && !e->cfg.float32 && n % 128 == 0 && k % 64 == 0;
}

__global__ void bf16_rows_to_f32_kernel(const bf16* src, const float* bias, float* dst, int n, long long total) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]) + (bias ? bias[i % n] : 0.0f);
}

__global__ void gate_up_bf16_kernel(const bf16* src, bf16* act, int ff, long long total) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ff, f = i % ff;
    const float g = __bfloat162float(src[r * 2 * ff + 2 * f]), u = __bfloat162float(src[r * 2 * ff + 2 * f + 1]);
    act[i] = __float2bfloat16_rn(gelu_tanh_f(g) * u);
  }
}

// out (fp32, or the gated activation) = EPI(a[rows, k] . w[n, k]^T)
template <typename T, int EPI>
int run_linear(mtx_layered* e, const void* a, const void* w, const float* bias, float* out, void* act, int rows, int n, int k, cudaStream_t st) {
  if (rows <= 0) return MTX_OK;
  LinArgs<T> p;
  memset(&p, 0, sizeof(p));
  p.a = static_cast<const T*>(a);
  p.w = static_cast<const T*>(w);
  p.bias = bias;
  p.out = out;
  p.act = static_cast<T*>(act);
  p.lda = k;
  p.ldo = EPI == LIN_GATED ? n / 2 : n;
  p.rows = rows;
  p.n = n;
  p.k = k;
  const dim3 grid((n + 63) / 64, (rows + 63) / 64);
  if constexpr (sizeof(T) == 4) return launch(linear_f32_kernel<EPI>, grid, dim3(kLinF32Threads), 0, st, p);
  else return launch(linear_mma_kernel<EPI>, grid, dim3(kLinThreads), 0, st, p);
}

// the same product on the tcgen05 GEMM: the bf16 result stays in e->obf (256-row blocks)
int run_umma_raw(mtx_layered* e, const void* a, const void* w, int rows, int n, int k, cudaStream_t st) {
  bf16* tmp = static_cast<bf16*>(e->obf);
  for (int r0 = 0; r0 < rows; r0 += 256) {
    const int nr = rows - r0 < 256 ? rows - r0 : 256;
    EpiArgs ea;
    memset(&ea, 0, sizeof(ea));
    ea.out = tmp + size_t(r0) * n;
    ea.ld_out = n;
    MTX_TRY(single_gemm<EPI_STORE_BF16>(static_cast<const bf16*>(a) + size_t(r0) * k, w, nr, n, k, ea, st));
  }
  return MTX_OK;
}

// ... then the epilogue as a row kernel
template <int EPI>
int run_linear_umma(mtx_layered* e, const void* a, const void* w, const float* bias, float* out, void* act, int rows, int n, int k, cudaStream_t st) {
  MTX_TRY(run_umma_raw(e, a, w, rows, n, k, st));
  const bf16* tmp = static_cast<const bf16*>(e->obf);
  const long long total = (long long)rows * (EPI == LIN_GATED ? n / 2 : n);
  const int blocks = int((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (EPI == LIN_GATED) return launch(gate_up_bf16_kernel, dim3(blocks), dim3(256), 0, st, tmp, static_cast<bf16*>(act), n / 2, total);
  return launch(bf16_rows_to_f32_kernel, dim3(blocks), dim3(256), 0, st, tmp, bias, out, n, total);
}

bool takes_umma(const mtx_layered* e, int rows, int n, int k) { return fits_umma(e, n, k) && rows >= 16; }

template <typename T, int EPI>
int linear(mtx_layered* e, const void* a, const void* w, const float* bias, float* out, void* act, int rows, int n, int k, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) {
    if (takes_umma(e, rows, n, k)) return run_linear_umma<EPI>(e, a, w, bias, out, act, rows, n, k, st);
  }
  return run_linear<T, EPI>(e, a, w, bias, out, act, rows, n, k, st);
}

int pick_key_tile(const mtx_layer_desc& l) {
  int kt = 32;
  while (kt > 4 && window_attn_smem_bytes(l.heads, l.kv_heads, l.dim, l.vdim, kt) > 200 * 1024) kt /= 2;
  return kt;
}

// x += gain * unit(a . w^T), and the copy of x in the matmul dtype
template <typename T>
int project_norm_residual(mtx_layered* e, const void* a, const void* w, int rows, int n, int k, float gain, cudaStream_t st) {
  const float* y = e->y;
  const bf16* yb = nullptr;
  if (sizeof(T) == 2 && takes_umma(e, rows, n, k)) {
    MTX_TRY(run_umma_raw(e, a, w, rows, n, k, st));
    y = nullptr;
    yb = static_cast<const bf16*>(e->obf);
  } else {
    MTX_TRY((linear<T, LIN_PLAIN>(e, a, w, nullptr, e->y, nullptr, rows, n, k, st)));
  }
  return launch(norm_residual_kernel<T>, dim3(rows), dim3(256), 0, st, y, yb, gain, e->cfg.eps, e->x, static_cast<T*>(e->xa), e->cfg.width);
}

bool use_window_mma() {
  static int on = env_int("MTX_WINDOW_MMA", 1);
  return on != 0;
}

template <int HPW, int DVT>
int launch_window_mma_t(const WindowAttnArgs<bf16>& wa, const WindowMmaExtra& x, size_t smem, cudaStream_t st) {
  static size_t have = 0;  // per instantiation
  if (smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(window_attention_mma_kernel<HPW, DVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  return launch(window_attention_mma_kernel<HPW, DVT>, dim3(x.n_tiles, x.splits), dim3(kWmmaThreads), smem, st, wa, x);
}

// the tensor-core mixer: (query tile, key split) work items, then the sum over the splits
int launch_window_mma(mtx_layered* e, const WindowAttnArgs<bf16>& wa, const WindowMmaPlan& plan, const mtx_ragged_batch& b, cudaStream_t st) {
  WindowMmaExtra x;
  x.tile_row0 = b.tile_row0;
  x.partial = e->attn_part;
  x.n_tiles = b.n_tiles;
  x.bn = plan.bn;
  x.hg = plan.hg;
  const int key_tiles = (wa.window + kWmmaRows - 1 + plan.bn - 1) / plan.bn;  // most key tiles a query tile can have
  // key splits: enough work items to fill the SMs (one CTA each), at least two key tiles per split, and among the next few counts
  // the one whose last wave is fullest (256 tiles x 2 splits on 148 SMs leave the fourth wave half empty; x 4 fill seven waves)
  int cap = key_tiles / 2;
  if (size_t(cap) * wa.rows > e->attn_part_rows) cap = int(e->attn_part_rows / wa.rows);
  if (cap < 1) cap = 1;
  int lo = (e->num_sms + b.n_tiles - 1) / b.n_tiles;
  if (lo > cap) lo = cap;
  int splits = lo;
  double best = 0.0;
  for (int sp = lo; sp <= cap && sp < lo + 8; ++sp) {
    const double waves = double(b.n_tiles) * sp / e->num_sms, eff = waves / std::ceil(waves);
    if (eff > best + 0.02) {
      best = eff;
      splits = sp;
    }
  }
  x.splits = splits;
  int rc = MTX_ERR_UNSUPPORTED;
  if (plan.hpw == 1 && plan.dvt == 8) rc = launch_window_mma_t<1, 8>(wa, x, plan.smem, st);
  else if (plan.hpw == 1 && plan.dvt == 16) rc = launch_window_mma_t<1, 16>(wa, x, plan.smem, st);
  else if (plan.hpw == 1 && plan.dvt == 32) rc = launch_window_mma_t<1, 32>(wa, x, plan.smem, st);
  else if (plan.hpw == 2 && plan.dvt == 8) rc = launch_window_mma_t<2, 8>(wa, x, plan.smem, st);
  else if (plan.hpw == 2 && plan.dvt == 16) rc = launch_window_mma_t<2, 16>(wa, x, plan.smem, st);
  MTX_TRY(rc);
  const long long per_split = (long long)wa.rows * wa.heads * wa.vdim;
  long long blocks = (per_split / 2 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch(window_partial_sum_kernel, dim3(unsigned(blocks)), dim3(256), 0, st, (const float*)e->attn_part, wa.out, splits, per_split);
}

template <int CPW, int DT>
int launch_window_decode_t(const WindowAttnArgs<bf16>& wa, const WindowDecodeExtra& x, size_t smem, cudaStream_t st) {
  static size_t have = 0;  // per instantiation
  if (smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(window_attention_decode_kernel<CPW, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  return launch(window_attention_decode_kernel<CPW, DT>, dim3(wa.rows, x.splits), dim3(kWdecThreads), smem, st, wa, x);
}

// the decode mixer (every row a token of its own sequence): (row, key split) work items, then the sum over the splits
int launch_window_decode(mtx_layered* e, const WindowAttnArgs<bf16>& wa, const WindowDecodePlan& plan, cudaStream_t st) {
  WindowDecodeExtra x;
  x.partial = e->attn_part;
  x.stages = plan.stages;
  const int key_tiles = (wa.window + kWdecKeys - 1) / kWdecKeys;
  // one wave: as many work items as CTAs fit on the GPU at once (a split's start-up -- its first tile's latency, the staging of
  // the queries -- is worth several tiles, so more and shorter splits lose), at least four key tiles per split
  size_t per_sm = (226 * 1024) / (plan.smem + 1024);
  if (per_sm > 8) per_sm = 8;
  int splits = int(per_sm) * e->num_sms / wa.rows;
  if (splits > key_tiles / 4) splits = key_tiles / 4;
  if (size_t(splits) * wa.rows > e->attn_part_rows) splits = int(e->attn_part_rows / wa.rows);
  if (splits < 1) splits = 1;
  x.splits = splits;
  int rc = MTX_ERR_UNSUPPORTED;
  if (plan.cpw == 1 && plan.dt == 4) rc = launch_window_decode_t<1, 4>(wa, x, plan.smem, st);
  else if (plan.cpw == 1 && plan.dt == 8) rc = launch_window_decode_t<1, 8>(wa, x, plan.smem, st);
  else if (plan.cpw == 1 && plan.dt == 16) rc = launch_window_decode_t<1, 16>(wa, x, plan.smem, st);
  else if (plan.cpw == 2 && plan.dt == 4) rc = launch_window_decode_t<2, 4>(wa, x, plan.smem, st);
  else if (plan.cpw == 2 && plan.dt == 8) rc = launch_window_decode_t<2, 8>(wa, x, plan.smem, st);
  MTX_TRY(rc);
  const long long per_split = (long long)wa.rows * wa.heads * wa.vdim;
  long long blocks = (per_split / 2 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch(window_partial_sum_kernel, dim3(unsigned(blocks)), dim3(256), 0, st, (const float*)e->attn_part, wa.out, splits, per_split);
}

bool use_window_decode() {
  static int on = env_int("MTX_WINDOW_DECODE", 1);
  return on != 0;
}

template <typename T>
int step_typed(mtx_layered* e, const mtx_ragged_batch& b, cudaStream_t st) {
  const mtx_layered_config& c = e->cfg;
  const int rows = b.rows, E = c.width;
  T* xa = static_cast<T*>(e->xa);
  MTX_TRY(launch(embed_rows_kernel<T>, dim3(rows), dim3(128), 0, st, b.token, static_cast<const T*>(c.embedding), c.vocab, c.embed_scale, e->x, xa, E));
  for (int li = 0; li < c.num_layers; ++li) {
    const mtx_layer_desc& l = e->layers[li];
    const int H = l.heads, G = l.kv_heads, nq = H * l.dim, nqkv = nq + G * l.dim + G * l.vdim, no = H * l.vdim;
    // q, k, v = W x + b
    QkvPostArgs<T> qa;
    memset(&qa, 0, sizeof(qa));
    if (sizeof(T) == 2 && takes_umma(e, rows, nqkv, E)) {  // the tcgen05 GEMM's bf16 result; the bias is added where it is read
      MTX_TRY(run_umma_raw(e, xa, l.wqkv, rows, nqkv, E, st));
      qa.qkv_bf16 = static_cast<const bf16*>(e->obf);
      qa.bias = l.bqkv;
    } else {
      if (l.bqkv) MTX_TRY((linear<T, LIN_BIAS>(e, xa, l.wqkv, l.bqkv, e->qkv, nullptr, rows, nqkv, E, st)));
      else MTX_TRY((linear<T, LIN_PLAIN>(e, xa, l.wqkv, nullptr, e->qkv, nullptr, rows, nqkv, E, st)));
      qa.qkv = e->qkv;
    }
    qa.q_norm = l.q_norm;
    qa.k_norm = l.k_norm;
    qa.q_out = static_cast<T*>(e->q);
    qa.k_pages = static_cast<T*>(l.k_pages);
    qa.v_pages = static_cast<T*>(l.v_pages);
    qa.v_shared = e->v_shared;
    qa.group = b.group;
    qa.pos = b.pos;
    qa.page_map = b.page_map;
    qa.heads = H;
    qa.kv_heads = G;
    qa.dim = l.dim;
    qa.vdim = l.vdim;
    qa.num_pages = c.num_pages;
    qa.tokens_per_page = c.tokens_per_page;
    qa.max_pages = c.max_pages_per_group;
    qa.value_mix = l.value_mix;
    qa.value_lambda = l.value_lambda;
    qa.eps = c.eps;
    MTX_TRY(launch(qkv_post_kernel<T>, dim3(rows), dim3(256), 0, st, qa));
    // the mixer
    WindowAttnArgs<T> wa;
    memset(&wa, 0, sizeof(wa));
    wa.q = static_cast<const T*>(e->q);
    wa.out = static_cast<T*>(e->attn);
    wa.k_pages = static_cast<const T*>(l.k_pages);
    wa.v_pages = static_cast<const T*>(l.v_pages);
    wa.group = b.group;
    wa.pos = b.pos;
    wa.page_map = b.page_map;
    wa.dist_bias = l.dist_bias;
    wa.head_bias = l.head_bias;
    wa.talk = l.talk;
    wa.rows = rows;
    wa.heads = H;
    wa.kv_heads = G;
    wa.dim = l.dim;
    wa.vdim = l.vdim;
    wa.window = l.window;
    wa.num_pages = c.num_pages;
    wa.tokens_per_page = c.tokens_per_page;
    wa.max_pages = c.max_pages_per_group;
    wa.scale = l.scale;
    wa.softcap = l.softcap;
    bool done = false;
    if constexpr (sizeof(T) == 2) {
      static const int force_stages = env_int("MTX_WINDOW_DECODE_STAGES", 0);
      const WindowDecodePlan dplan = window_decode_plan(H, G, l.dim, l.vdim, force_stages);
      const WindowMmaPlan plan = window_mma_plan(H, G, l.dim, l.vdim);
      if (dplan.ok && b.n_tiles == rows && b.tile_row0 != nullptr && use_window_mma() && use_window_decode()) {  // all single-row tiles
        MTX_TRY(launch_window_decode(e, wa, dplan, st));
        done = true;
      } else if (plan.ok && b.n_tiles > 0 && b.tile_row0 != nullptr && use_window_mma()) {
        MTX_TRY(launch_window_mma(e, wa, plan, b, st));
        done = true;
      }
    }
    if (!done) {
      wa.kt = pick_key_tile(l);
      const size_t smem = window_attn_smem_bytes(H, G, l.dim, l.vdim, wa.kt);
      static size_t attr_bytes[2] = {0, 0};  // per instantiation (bf16, float)
      size_t& have = attr_bytes[sizeof(T) == 4 ? 1 : 0];
      if (smem > 48 * 1024 && smem > have) {
        MTX_CUDA(cudaFuncSetAttribute(window_attention_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        have = smem;
      }
      MTX_TRY(launch(window_attention_rows_kernel<T>, dim3(rows), dim3(kWinThreads), smem, st, wa));
    }
    // x += gain1 * unit(Wo attn)
    MTX_TRY(project_norm_residual<T>(e, e->attn, l.wo, rows, E, no, l.gain1, st));
    if (l.ff > 0) {
      // x += gain2 * unit(Wdown (gelu(Wgate x) * Wup x))
      MTX_TRY((linear<T, LIN_GATED>(e, xa, l.w_gate_up, nullptr, nullptr, e->act, rows, 2 * l.ff, E, st)));
      MTX_TRY(project_norm_residual<T>(e, e->act, l.w_down, rows, E, l.ff, l.gain2, st));
    }
  }
  if (b.n_want > 0) {
    T* wn = static_cast<T*>(e->wanted);
    MTX_TRY(launch(scalar_norm_rows_kernel<T>, dim3(b.n_want), dim3(256), 0, st, (const float*)e->x, b.want_rows, c.final_gain, c.eps, wn, E));
    MTX_TRY((linear<T, LIN_PLAIN>(e, wn, c.head, nullptr, b.logits, nullptr, b.n_want, c.vocab, E, st)));
  }
  return MTX_OK;
}

}  // namespace

extern "C" {

int mtx_layered_create(const mtx_layered_config* cfg, const mtx_layer_desc* layers, mtx_layered** out) {
  if (!cfg || !layers || !out) return fail(MTX_ERR_ARG, "null argument");
  const mtx_layered_config& c = *cfg;
  if (c.num_layers < 1 || c.width < 1 || c.vocab < 1 || c.max_rows < 1 || c.max_want < 0) return fail(MTX_ERR_ARG, "bad layer count / width / vocab / rows");
  if (c.num_groups < 1 || c.num_pages < 2 || c.tokens_per_page < 1 || c.max_pages_per_group < 1) return fail(MTX_ERR_ARG, "bad page geometry");
  if (!c.embedding || !c.head) return fail(MTX_ERR_ARG, "embedding / head missing");
  mtx_layered* e = new mtx_layered();
  e->cfg = c;
  e->layers.assign(layers, layers + c.num_layers);
  int first_mix = -1;
  for (int i = 0; i < c.num_layers; ++i) {
    const mtx_layer_desc& l = e->layers[i];
    int rc = MTX_OK;
    if (l.mixer != MTX_MIXER_WINDOW_SIGMOID) rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: unknown mixer %d", i, l.mixer);
    else if (l.heads < 1 || l.kv_heads < 1 || l.heads % l.kv_heads != 0 || l.dim < 1 || l.vdim < 1 || l.window < 1 || l.ff < 0)
      rc = fail(MTX_ERR_ARG, "layer %d: bad head geometry / window / ff", i);
    else if (l.heads * l.vdim > kWinThreads * kWinMaxAcc)
      rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: heads * vdim = %d exceeds %d", i, l.heads * l.vdim, kWinThreads * kWinMaxAcc);
    else if (window_attn_smem_bytes(l.heads, l.kv_heads, l.dim, l.vdim, 4) > 200 * 1024)
      rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: the heads do not fit the attention kernel's shared memory", i);
    else if (!l.wqkv || !l.wo || !l.dist_bias || !l.k_pages || !l.v_pages || (l.ff > 0 && (!l.w_gate_up || !l.w_down)))
      rc = fail(MTX_ERR_ARG, "layer %d: a weight or a page pool is missing", i);
    else if (l.value_mix < 0 || l.value_mix > 2) rc = fail(MTX_ERR_ARG, "layer %d: value_mix must be 0, 1 or 2", i);
    if (rc == MTX_OK && l.value_mix == 1) {
      if (first_mix >= 0) rc = fail(MTX_ERR_ARG, "layer %d: only one layer keeps its values for the others", i);
      first_mix = i;
      e->vshared_dim = l.kv_heads * l.vdim;
    }
    if (rc == MTX_OK && l.value_mix == 2 && (first_mix < 0 || l.kv_heads * l.vdim != e->vshared_dim))
      rc = fail(MTX_ERR_ARG, "layer %d mixes in the values of an earlier layer: none kept them, or their size differs", i);
    if (rc != MTX_OK) {
      delete e;
      return rc;
    }
    const int nqkv = l.heads * l.dim + l.kv_heads * (l.dim + l.vdim);
    if (nqkv > e->max_nqkv) e->max_nqkv = nqkv;
    if (l.heads * l.dim > e->max_qdim) e->max_qdim = l.heads * l.dim;
    if (l.heads * l.vdim > e->max_odim) e->max_odim = l.heads * l.vdim;
    if (2 * l.ff > e->max_nqkv) e->max_nqkv = 2 * l.ff;  // (the tcgen05 path parks the gate / up product in the same scratch)
    if (l.ff > e->max_ff) e->max_ff = l.ff;
  }
  if (c.vocab > e->max_nqkv) e->max_nqkv = c.vocab;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) e->num_sms = sms;
  cudaGetLastError();
  e->ws_bytes = layered_layout(e).total;
  *out = e;
  return MTX_OK;
}

int mtx_layered_destroy(mtx_layered* e) {
  if (e == nullptr) return MTX_OK;
  for (auto& g : e->graphs) cudaGraphExecDestroy(g.exec);
  if (e->cap_stream) cudaStreamDestroy(e->cap_stream);
  delete e;
  return MTX_OK;
}

size_t mtx_layered_workspace_bytes(const mtx_layered* e) { return e ? e->ws_bytes : 0; }

int mtx_layered_bind(mtx_layered* e, void* workspace, size_t workspace_bytes) {
  if (!e || !workspace) return fail(MTX_ERR_ARG, "null argument");
  if (workspace_bytes < e->ws_bytes) return fail(MTX_ERR_ARG, "workspace of %zu bytes, %zu needed", workspace_bytes, e->ws_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 1023) != 0) return fail(MTX_ERR_ARG, "the workspace must be 1024-byte aligned");
  const LWs L = layered_layout(e);
  char* base = static_cast<char*>(workspace);
  e->x = reinterpret_cast<float*>(base + L.x);
  e->y = reinterpret_cast<float*>(base + L.y);
  e->qkv = reinterpret_cast<float*>(base + L.qkv);
  e->v_shared = reinterpret_cast<float*>(base + L.v_shared);
  e->xa = base + L.xa;
  e->q = base + L.q;
  e->attn = base + L.attn;
  e->act = base + L.act;
  e->wanted = base + L.wanted;
  e->obf = base + L.obf;
  e->attn_part = reinterpret_cast<float*>(base + L.attn_part);
  e->attn_part_rows = 4 * align_up(size_t(e->cfg.max_rows), 256);
  e->bound = true;
  return MTX_OK;
}

int mtx_layered_step(mtx_layered* e, const mtx_ragged_batch* b, mtx_stream stream) {
  if (!e || !e->bound || !b) return fail(MTX_ERR_ARG, "engine is not bound / null argument");
  if (b->rows < 1 || b->rows > e->cfg.max_rows) return fail(MTX_ERR_ARG, "rows = %d outside [1, %d]", b->rows, e->cfg.max_rows);
  if (b->n_want < 0 || b->n_want > e->cfg.max_want) return fail(MTX_ERR_ARG, "n_want = %d outside [0, %d]", b->n_want, e->cfg.max_want);
  if (!b->token || !b->group || !b->pos || !b->page_map || (b->n_want > 0 && (!b->want_rows || !b->logits))) return fail(MTX_ERR_ARG, "null batch array");
  if (b->n_tiles < 0 || b->n_tiles > b->rows) return fail(MTX_ERR_ARG, "n_tiles = %d for %d rows", b->n_tiles, b->rows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return e->cfg.float32 ? step_typed<float>(e, *b, st) : step_typed<bf16>(e, *b, st);
}

int mtx_layered_step_graph(mtx_layered* e, const mtx_ragged_batch* b, mtx_stream stream) {
  if (!e || !e->bound || !b) return fail(MTX_ERR_ARG, "engine is not bound / null argument");
  for (auto& g : e->graphs) {
    if (memcmp(&g.key, b, sizeof(*b)) == 0) {
      MTX_CUDA(cudaGraphLaunch(g.exec, static_cast<cudaStream_t>(stream)));
      return MTX_OK;
    }
  }
  if (e->graphs.size() >= 64) return mtx_layered_step(e, b, stream);  // (a caller that never repeats a descriptor)
  if (!e->cap_stream) MTX_CUDA(cudaStreamCreateWithFlags(&e->cap_stream, cudaStreamNonBlocking));
  cudaGraph_t graph = nullptr;
  MTX_CUDA(cudaStreamBeginCapture(e->cap_stream, cudaStreamCaptureModeThreadLocal));
  const int rc = mtx_layered_step(e, b, e->cap_stream);
  const cudaError_t end = cudaStreamEndCapture(e->cap_stream, &graph);
  if (rc != MTX_OK) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (end != cudaSuccess) return fail(MTX_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(end));
  cudaGraphExec_t exec = nullptr;
  const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (inst != cudaSuccess) return fail(MTX_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(inst));
  mtx_layered::GraphEntry ge;
  memcpy(&ge.key, b, sizeof(*b));
  ge.exec = exec;
  e->graphs.push_back(ge);
  MTX_CUDA(cudaGraphLaunch(exec, static_cast<cudaStream_t>(stream)));
  return MTX_OK;
}

}  // extern "C"
