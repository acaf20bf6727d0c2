// Host-side plumbing shared by the translation units of the library: error reporting, TMA descriptors, the kernel launch helper
// (programmatic dependent launch, clusters, optional per-launch timing) and the launchers of the tcgen05 GEMMs.
#pragma once

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/mtx_b200.h"
#include "gemm_rows.cuh"
#include "gemm_umma.cuh"

namespace mtx {
// one instance per library, whichever translation unit touches it
inline thread_local std::string g_error;
inline std::atomic<uint64_t> g_launches{0};
}  // namespace mtx

using namespace mtx;

namespace {


int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

#define MTX_CUDA(expr)                                                                          \
  do {                                                                                          \
    cudaError_t err__ = (expr);                                                                 \
    if (err__ != cudaSuccess) return fail(MTX_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)

#define MTX_TRY(expr)            \
  do {                           \
    int rc__ = (expr);           \
    if (rc__ != MTX_OK) return rc__; \
  } while (0)

int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
}

// ---- TMA descriptors ---------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 matrix [outer, inner] (inner contiguous), box [box_outer, 64] with the 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint32_t box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(MTX_ERR_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (inner * 2) % 16 != 0)
    return fail(MTX_ERR_ARG, "TMA needs a 16-byte aligned base and row pitch");
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner * 2};
  const cuuint32_t box[2] = {64, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(MTX_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(rc));
  return MTX_OK;
}

// uint8 matrix [outer, 64] (one int8 cache row of a kv head per matrix row), box [64, 64] with the 64-byte swizzle.
int make_map_u8(CUtensorMap* m, const void* base, uint64_t outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(MTX_ERR_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(MTX_ERR_ARG, "TMA needs a 16-byte aligned base");
  const cuuint64_t dims[2] = {64, outer};
  const cuuint64_t strides[1] = {64};
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(MTX_ERR_CUDA, "cuTensorMapEncodeTiled (uint8) failed with CUresult %d", int(rc));
  return MTX_OK;
}

// ---- launch helper -------------------------------------------------------------------------

// Optional per-kernel timing: when a sink is installed every launch is bracketed by CUDA
// events on the launching stream and attributed to the current kernel class.
enum KernelClass { KC_PREPARE = 0, KC_RMSNORM, KC_QKV, KC_ATTENTION, KC_OUTPROJ, KC_MLP_UP, KC_MLP_DOWN, KC_LOGITS, KC_FINALIZE, KC_PERSISTENT, KC_COUNT };
struct ProfileSink {
  struct Rec { int cls; cudaEvent_t a, b; };
  std::vector<Rec> recs;
};
thread_local ProfileSink* g_profile = nullptr;
thread_local int g_class = KC_PREPARE;
long long* g_trace = nullptr;  // debug timeline buffer (device), see mtx_debug_set_trace

bool use_pdl() {
  static int v = env_int("MTX_PDL", 1);
  return v != 0;
}

thread_local int g_cluster_y = 1;  // cluster size along grid.y for the next launch (split-K GEMM)
thread_local bool g_cooperative = false;  // next launch is cooperative: all its CTAs are co-resident or the launch fails

template <typename... KArgs, typename... Args>
int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (g_cooperative) {
    attr[na].id = cudaLaunchAttributeCooperative;
    attr[na].val.cooperative = 1;
    ++na;
  } else if (use_pdl()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (g_cluster_y > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = unsigned(g_cluster_y);
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  ProfileSink::Rec rec;
  if (g_profile != nullptr) {
    rec.cls = g_class;
    MTX_CUDA(cudaEventCreate(&rec.a));
    MTX_CUDA(cudaEventCreate(&rec.b));
    MTX_CUDA(cudaEventRecord(rec.a, stream));
  }
  MTX_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
  if (g_profile != nullptr) {
    MTX_CUDA(cudaEventRecord(rec.b, stream));
    g_profile->recs.push_back(rec);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return MTX_OK;
}

// Attention work items the per-kernel path aims for: a multiple of the SM count, so that the (at most 3 per SM) persistent CTAs
// of decode_attn_kernel each walk several items and finish together (with one item per (row, kv head) pair, batch 256 leaves
// 1024 whole-sequence items for 444 CTAs: two or three each, a 30 % imbalance).
int attn_target_items(int num_sms) { return num_sms * env_int("MTX_ATTN_ITEMS_PER_SM", 1); }

int round_rows(int rows) {
  int t = 16;
  while (t < rows) t *= 2;
  return t;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct GemmPlan {
  int n_tiles, splits, stages;
  size_t smem;
};

// K splits = cluster size: a power of two <= 16 (8 is the portable maximum, 16 needs the
// non-portable opt-in), chosen so that n_tiles * splits is close to one CTA per SM.
GemmPlan plan_gemm(int n, int k, int r_tile, int num_sms, int epi, int forced_splits = 0) {
  GemmPlan g;
  g.n_tiles = (n + kTileN - 1) / kTileN;
  const int kb = k / kBlockK;
  int splits = forced_splits;
  if (splits <= 0) {
    const int target = env_int("MTX_GEMM_TARGET_CTAS", num_sms);
    const int max_split = env_int("MTX_GEMM_MAX_SPLIT", 16);
    const double want = double(target) / g.n_tiles;
    splits = 1;
    while (splits * 2 <= max_split && splits * 2 <= kb && splits * 2 <= r_tile && double(splits) * 1.42 < want) splits *= 2;
  }
  g.splits = splits;
  const int stage_bytes = kWTileBytes + r_tile * kBlockK * 2;
  const int budget = (r_tile <= 128 ? 100 : 200) * 1024;
  int stages = budget / stage_bytes;
  const int max_kb = (kb + splits - 1) / splits;
  if (stages > max_kb) stages = max_kb;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 1) stages = 1;
  g.stages = stages;
  g.smem = gemm_smem_bytes(stages, r_tile, splits, epi);
  return g;
}

template <int EPI>
int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, GemmParams p, const EpiArgs& e, const GemmPlan& g, cudaStream_t st) {
  static bool attr_set = false;  // per template instance
  if (!attr_set) {
    MTX_CUDA(cudaFuncSetAttribute(gemm_umma_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    MTX_CUDA(cudaFuncSetAttribute(gemm_umma_kernel<EPI>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    attr_set = true;
  }
  p.splits = g.splits;
  p.stages = g.stages;
  p.trace = g_trace;
  g_cluster_y = g.splits;
  const int rc = launch(gemm_umma_kernel<EPI>, dim3(g.n_tiles, g.splits), dim3(kGemmThreads), g.smem, st, tw, tx, p, e);
  g_cluster_y = 1;
  return rc;
}

// ---- steps of 65..256 rows: gemm_rows.cuh ------------------------------------------------------
struct RowsPlan {
  int n_tiles, splits, stages, grid_x, row_blocks, r_tile_cta;
  size_t smem;
};

RowsPlan plan_rows(int n, int k, int r_tile, int num_sms, int epi, int forced_splits = 0) {
  RowsPlan g;
  g.n_tiles = (n + kTileN - 1) / kTileN;
  const int kb = k / kBlockK;
  int splits = forced_splits;
  if (splits <= 0) {
    splits = 1;
    // few tiles: cut K over a cluster of up to 8 CTAs (the portable maximum; two such clusters fit a GPC) until the
    // grid covers most of the SMs.  Many tiles: one persistent CTA per SM walks them with double-buffered accumulators.
    // (a split unit covers one 128-row block, and two units fit one SM: up to 1.25 units per SM)
    if (epi != EPI_LOGITS && g.n_tiles * 2 <= num_sms) {
      const int max_split = env_int("MTX_ROWS_MAX_SPLIT", 8);
      const int zb = r_tile / 128;
      while (splits * 2 <= max_split && splits * 2 <= kb && g.n_tiles * zb * splits * 2 <= num_sms + num_sms / 4) splits *= 2;
    }
  }
  g.splits = splits;
  g.row_blocks = splits > 1 ? r_tile / 128 : 1;
  g.r_tile_cta = splits > 1 ? 128 : r_tile;
  r_tile = g.r_tile_cta;
  const int stage_bytes = kWTileBytes + r_tile * kBlockK * 2;
  int stages = ((splits > 1 ? 96 : 192) * 1024) / stage_bytes;
  const int max_kb = splits > 1 ? (kb + splits - 1) / splits : kb * 2;
  if (stages > max_kb) stages = max_kb;
  if (stages > kRowsMaxStages) stages = kRowsMaxStages;
  if (stages < 1) stages = 1;
  g.stages = stages;
  g.grid_x = splits > 1 ? g.n_tiles : (g.n_tiles < num_sms ? g.n_tiles : num_sms);
  g.smem = rows_smem_bytes(stages, r_tile, splits);
  return g;
}

template <int EPI>
int launch_rows(const CUtensorMap& tw, const CUtensorMap& tx, GemmParams p, const EpiArgs& e, const RowsPlan& g, cudaStream_t st) {
  static bool attr_set = false;  // per template instance
  if (!attr_set) {
    MTX_CUDA(cudaFuncSetAttribute(gemm_rows_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
  p.splits = g.splits;
  p.stages = g.stages;
  p.r_tile = g.r_tile_cta;
  p.trace = g_trace;
  g_cluster_y = g.splits;
  const int rc = launch(gemm_rows_kernel<EPI>, dim3(g.grid_x, g.splits, g.row_blocks), dim3(kRowsThreads), g.smem, st, tw, tx, p, e);
  g_cluster_y = 1;
  return rc;
}

bool use_rows_kernel(int r_tile) {
  static int on = env_int("MTX_ROWS_KERNEL", 1);
  return on != 0 && r_tile >= 128;
}

// (plan_gemm / launch_gemm are declared above)
// out = EPI(x[rows, k] . w[n, k]^T) on whichever tcgen05 GEMM serves the row count (gemm_umma.cuh up to 64 rows, gemm_rows.cuh above)
template <int EPI>
int single_gemm(const void* x, const void* w, int rows, int n, int k, EpiArgs ea, cudaStream_t st) {
  const int r_tile = round_rows(rows);
  CUtensorMap tw, tx;
  MTX_TRY(make_map(&tw, w, k, n, kTileN));
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.n = n;
  p.k = k;
  p.rows = rows;
  p.r_tile = r_tile;
  if (use_rows_kernel(r_tile)) {
    const RowsPlan pl = plan_rows(n, k, r_tile, 148, EPI);
    MTX_TRY(make_map(&tx, x, k, r_tile, pl.splits > 1 ? 128 : r_tile));
    return launch_rows<EPI>(tw, tx, p, ea, pl, st);
  }
  MTX_TRY(make_map(&tx, x, k, r_tile, r_tile));
  return launch_gemm<EPI>(tw, tx, p, ea, plan_gemm(n, k, r_tile, 148, EPI), st);
}

}  // namespace
